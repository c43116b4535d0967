"""bin/trace_run end to end on a Nununex model from files: a config.json and a model.safetensors written by the test
(every tensor name of the design: all three mixers, both feed-forwards, a layer without one, a decay projection and a
distance-bias table whose sizes only the checkpoint gives), a schedule on standard input with portions beside single
tokens and requests that end and give their pages and state slots to later ones, logits compared with the CPU oracle."""
import json
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from nununex_common import clean, dense, gdelta, model_cfg, moe, par, random_checkpoint, scan, write_checkpoint

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def default_config():
    # eps far below the read-outs' squares: a request of ONE token reads o = (r . k) v from the delta rule's empty state,
    # and when r . k happens to be small, an eps of its size would turn the product's rounding into an error of the norm
    return model_cfg([
        (gdelta(2, 14), moe(4, 2, 10, 12)),
        (par(3, 1, 12, 8, window=11, bias_max=30, rows=10, scale=0.4, mheads=2, mdim=6, mvdim=10, cap=7.0), dense(26)),
        (scan(18, 5, 2, 3), None),
        (par(2, 2, 8, 10, window=70, bias_max=20, rows=6, mheads=1, mdim=8, mvdim=8), dense(18)),
    ], vocab=50, width=36, eps=1e-8, taps=4, cap=20.0, buckets=41, mul_prev=13, mul_cur=5, decay_rank=7)


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 8e-2)])
def test_trace_run_replays_a_schedule_from_files(tmp_path, dtype, tol):
    from oracle import nununex as O

    cfg = default_config()
    tensors = random_checkpoint(cfg, seed=3)
    write_checkpoint(tmp_path / "model", cfg, tensors)
    c = clean(cfg)
    g = torch.Generator().manual_seed(5)
    reqs = {k: torch.randint(0, 50, (n,), generator=g).tolist() for k, n in (("a", 40), ("b", 17), ("c", 5), ("d", 70), ("e", 1))}
    want = {k: O.forward(c, tensors, v) for k, v in reqs.items()}
    # pool: 3 pages of 64 tokens; a, b, c live together, then d (2 pages) beside b after a and c have ended, then e
    plan = [[("a", 16), ("b", 2)], [("a", 1), ("b", 1)], [("a", 23), ("c", 5)], [("b", 1)], [("b", 13), ("d", 33)],
            [("d", 1)], [("d", 36), ("e", 1)]]
    at = {k: 0 for k in reqs}
    lines, expect = [], []
    for n, step in enumerate(plan):
        entries, end, rows = [], [], []
        for k, cnt in step:
            lo, hi = at[k], at[k] + cnt
            entries.append({"id": "req-" + k, "tokens": reqs[k][lo:hi], "want": list(range(cnt))})
            rows.append(want[k][lo:hi])
            at[k] = hi
            if hi == len(reqs[k]):
                end.append("req-" + k)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
        expect.append(torch.cat(rows))
    assert all(at[k] == len(v) for k, v in reqs.items())
    out = tmp_path / "out"
    env = dict(os.environ, HOME=str(tmp_path), TMPDIR=str(tmp_path))
    res = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(tmp_path / "model"), "--dtype", dtype, "--out",
                          str(out), "--max-tokens", "192"], input="\n".join(lines) + "\n", capture_output=True, text=True,
                         env=env, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
    scale = torch.cat(list(want.values())).std()
    errs = []
    for n, exp in enumerate(expect):
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(exp.shape)).double()
        d = (got - exp) - (got - exp).mean(-1, keepdim=True)
        errs.append(d.pow(2).mean(-1).sqrt() / scale)
    errs = torch.cat(errs)
    assert errs.max() < tol
