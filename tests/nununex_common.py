"""Helpers of the Nununex tests: small configurations, checkpoints with random tensors under the design's names, a
runner that holds them."""
import json
import struct
from pathlib import Path

import torch


def gdelta(heads=3, dim=12):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}}


def par(heads=4, kv_heads=2, dim=12, vdim=10, window=7, bias_max=24, rows=8, scale=None, mheads=3, mdim=8, mvdim=12,
        cap=9.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 1.3 * dim ** -0.5,
            "bias_max": bias_max, "mask": {"size": window}, "_rows": rows}
    right = {"heads": mheads, "dim": mdim, "vdim": mvdim, "gate_cap": cap}
    return {"type": "parallel", "mixer": {"left": left, "right": right}}


def scan(inner=24, state=6, dt_rank=3, conv=3):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=12, shared=20):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def model_cfg(layers, vocab=83, width=48, eps=1e-5, taps=3, cap=12.0, buckets=61, mul_prev=29, mul_cur=7, decay_rank=5):
    """`_rows` (rows of a layer's distance-bias table) and `_decay_rank` are not keys of the design's config.json:
    the checkpoint's tensors carry them; `random_checkpoint` reads them from here."""
    return {"architecture": "Nununex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "logit_softcap": cap, "_decay_rank": decay_rank,
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
            "layers": [dict(mixer_layer, mlp=mlp) for mixer_layer, mlp in layers]}


def config_a():
    """All three mixers, both feed-forwards, a layer without one; odd sizes (the kernels' scalar paths)."""
    return model_cfg([
        (scan(24, 6, 3, 3), dense(40)),
        (gdelta(3, 12), moe(5, 2, 12, 20)),
        (par(4, 2, 12, 10, window=7, bias_max=24, rows=8, mheads=3, mdim=8, mvdim=12), None),
        (gdelta(2, 20), dense(28)),
        (par(3, 3, 10, 14, window=19, bias_max=12, rows=6, mheads=2, mdim=12, mvdim=6), moe(4, 1, 16, 0)),
        (scan(20, 9, 2, 4), moe(6, 3, 8, 16)),
    ])


def config_b():
    """Sizes in multiples of 16: the vector and tensor-core paths of the attention kernels."""
    return model_cfg([
        (par(4, 2, 32, 32, window=21, bias_max=64, rows=16, mheads=2, mdim=32, mvdim=32), dense(64)),
        (gdelta(2, 32), moe(8, 2, 16, 32)),
        (scan(64, 16, 4, 4), dense(48)),
        (par(2, 1, 64, 64, window=40, bias_max=100, rows=12, mheads=4, mdim=16, mvdim=16), None),
    ], vocab=96, width=64, eps=1e-6, taps=4, cap=30.0, buckets=127, mul_prev=1000003, mul_cur=31, decay_rank=8)


def random_checkpoint(cfg: dict, seed: int = 0) -> dict:
    """Every tensor name of the design with random bfloat16 values, for the given config.json dict."""
    W, V, taps = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    g = torch.Generator().manual_seed(seed)
    t = {}

    def mat(name, *shape, scale=None):
        t[name] = (torch.randn(*shape, generator=g) * (scale if scale is not None else shape[-1] ** -0.5)).to(torch.bfloat16)

    def vec(name, *shape, mean=0.0, spread=0.1):
        t[name] = (mean + spread * torch.randn(*shape, generator=g)).to(torch.bfloat16)

    mat("embed", V, W, scale=1.0)
    mat("bigram", cfg["embedding"]["bigram"]["buckets"] + 1, W, scale=0.5)
    mat("head", V, W, scale=2.0 * W ** -0.5)
    vec("final.norm", W, mean=1.0)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        subs = ("1", "2") if layer.get("mlp") is not None else ("1",)
        for s in subs:
            vec(p + "norm" + s, W, mean=1.0)
            mat(p + "canon" + s, W, taps, scale=0.4)
            mat(p + "rg" + s, W, W)
            vec(p + "rg" + s + ".b", W, mean=0.5, spread=0.5)
        q = p + "mix."
        if layer["type"] == "general_delta":
            H, D, R = m["heads"], m["dim"], cfg.get("_decay_rank", 5)
            for n in "rkvga":
                mat(q + n, H * D, W)
            vec(q + "a.b", H * D, spread=0.5)
            mat(q + "w1", R, W)
            mat(q + "w2", H * D, R, scale=1.0)
            vec(q + "w0", H * D, spread=1.0)
            vec(q + "norm", H * D, mean=1.0)
            mat(q + "o", W, H * D)
        elif layer["type"] == "parallel":
            a, r = m["left"], m["right"]
            H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            mat(q + "left.q", H * D, W); mat(q + "left.k", G * D, W); mat(q + "left.v", G * Dv, W)
            vec(q + "left.rel", a.get("_rows", 8), H, spread=1.0)
            vec(q + "left.sink", H, spread=1.0)
            mat(q + "left.o", W, H * Dv)
            vec(q + "left.out", W, mean=1.0)
            H, D, Dv = r["heads"], r["dim"], r["vdim"]
            mat(q + "right.q", H * D, W); mat(q + "right.k", H * D, W); mat(q + "right.v", H * Dv, W)
            mat(q + "right.g", H * Dv, W)
            mat(q + "right.i", H, W, scale=2.0 * W ** -0.5); vec(q + "right.i.b", H, spread=1.0)
            mat(q + "right.f", H, W, scale=2.0 * W ** -0.5); vec(q + "right.f.b", H, mean=2.0, spread=1.0)
            vec(q + "right.norm", H * Dv, mean=1.0)
            mat(q + "right.o", W, H * Dv)
            vec(q + "right.out", W, mean=1.0)
        else:
            inner, S, R, ct = m["inner"], m["state"], m["dt_rank"], m["conv"]
            mat(q + "in", 2 * inner, W)
            mat(q + "conv", inner, ct, scale=0.5); vec(q + "conv.b", inner)
            mat(q + "x", R + 2 * S, inner)
            mat(q + "dt", inner, R, scale=1.0); vec(q + "dt.b", inner, mean=-1.0, spread=0.5)
            vec(q + "A_log", inner, S, spread=0.7)
            vec(q + "D", inner, mean=1.0)
            mat(q + "o", W, inner)
        f, mlp = p + "mlp.", layer.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            mat(f + "up", mlp["ff"], W); vec(f + "up.b", mlp["ff"])
            mat(f + "down", W, mlp["ff"]); vec(f + "down.b", W)
        else:
            ff = mlp["expert"]["ff"]
            mat(f + "router", mlp["router"]["experts"], W, scale=3.0 * W ** -0.5)    # scores spread over (0, 1)
            for e in range(mlp["router"]["experts"]):
                mat(f + f"e{e}.gate", ff, W); mat(f + f"e{e}.up", ff, W); mat(f + f"e{e}.down", W, ff)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                mat(f + "shared.gate", sf, W); mat(f + "shared.up", sf, W); mat(f + "shared.down", W, sf)
                mat(f + "shared.sg", 1, W)
    return t


def clean(cfg: dict) -> dict:
    """The config.json as a checkpoint folder holds it: without the helpers' private keys."""
    c = json.loads(json.dumps(cfg))
    c.pop("_decay_rank", None)
    for layer in c["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["left"].pop("_rows", None)
    return c


def make_runner(cfg_json, tensors=None, dtype="float32", pages=24, page_size=16, max_seqs=4, seed=0,
                max_batched_tokens=None, device_allocator=False, eager=True):
    """A runner for the configuration; `tensors` (checkpoint names) are loaded over the synthetic weights."""
    from compactor_vllm.config.engine_config import LLMConfig
    from compactor_vllm.config.model_config import NununexConfig
    from compactor_vllm.core.model_runner import ModelRunner

    hf = NununexConfig.from_json(clean(cfg_json))
    cfg = LLMConfig(model="synthetic", hf_config=hf, dtype=dtype, max_num_seqs=max_seqs, kvcache_page_size=page_size,
                    max_model_len=pages * page_size, enforce_eager=eager)
    r = ModelRunner(cfg, num_pages=pages, seed=seed, device_allocator=device_allocator,
                    max_batched_tokens=max_batched_tokens)
    if tensors is not None:
        r.model.load_weights(tensors)
    return r


def build(cfg_json, dtype="float32", seed=0, **kw):
    """(runner, clean config, tensors) of a random model."""
    tensors = random_checkpoint(cfg_json, seed)
    return make_runner(cfg_json, tensors, dtype, **kw), clean(cfg_json), tensors


def write_checkpoint(folder: Path, cfg: dict, tensors: dict) -> None:
    header, blob = {}, b""
    for name, x in tensors.items():
        raw = x.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(x.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    h = json.dumps(header).encode()
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(clean(cfg)))
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + blob)


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def row_errs(got, want):
    """Per row: rms of the centred difference over the rms of the centred expectation."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()


def rel_err(got, want):
    return row_errs(got, want).max().item()


TOL = {"float32": 3e-5, "bfloat16": 6e-2}


def close(got, want, dtype):
    e = row_errs(got, want).flatten()
    if dtype == "float32":
        return bool(e.max() < TOL[dtype])
    return bool(e.median() < 0.03 and e.max() < 0.15)


def new_seq():
    from compactor_vllm.utils.sequence import Sequence

    return Sequence(prompt_token_ids=[])


def feed(runner, seq, toks, all_rows=True):
    seq.prompt_token_ids.extend(toks)
    return runner.run_step([(seq, toks)], rows=list(range(len(toks))) if all_rows else None)


def run_in_portions(runner, toks, sizes):
    """The request alone, cut into portions of the given sizes (cycled); logits of every position."""
    seq, out, at, k = new_seq(), [], 0, 0
    while at < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - at)
        out.append(feed(runner, seq, toks[at:at + n]))
        at, k = at + n, k + 1
    runner.release([seq])
    return torch.cat(out)
