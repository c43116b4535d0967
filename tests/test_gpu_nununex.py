"""Nununex through the engine against the plain CPU oracle (oracle/nununex.py).

Every test makes its own small configuration and random weights (checkpoint tensors under the design's names, loaded
by the model's `load_weights`).  The engine runs them through its runner (`ModelRunner.run_step`, the paged cache, the
state pool, the native kernels); the oracle recomputes whole sequences without a cache or a carried state.  float32
runs are compared sharply (they show a key that is one position off, a lost state or a missing sink), bfloat16 loosely."""
import math

import pytest
import torch

from nununex_common import (TOL, build, close, config_a, config_b, dense, feed, gdelta, model_cfg, moe, new_seq, par,
                            rel_err, run_in_portions, scan, tokens)

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


# ------------------------------------------------------------------------------------------ mechanisms one by one
@pytest.mark.parametrize("width", [40, 257, 1024])
def test_gated_residual_sum_and_norm(width):
    from compactor_vllm.layers.layernorm import gated_residual_norm
    from oracle import nununex as O

    g = torch.Generator().manual_seed(1)
    x = torch.randn(7, width, generator=g) * 3
    w = 1 + 0.2 * torch.randn(width, generator=g)
    for ydt, gdt in ((torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16), (torch.float32, torch.float32)):
        y = torch.randn(7, width, generator=g).to(ydt)
        z = (2 * torch.randn(7, width, generator=g)).to(gdt)
        want_x = x.double() + O.sigmoid(z.double()) * y.double()
        xr = x.clone().to(DEV)
        h = gated_residual_norm(xr, branch=y.to(DEV), gate=z.to(DEV), weight=w.to(DEV), eps=1e-5, out_dtype=torch.float32)
        assert torch.allclose(xr.cpu().double(), want_x, rtol=1e-6, atol=1e-6)
        assert torch.allclose(h.cpu().double(), O.rms_unit(want_x, 1e-5) * w.double(), rtol=2e-5, atol=2e-5)
        assert gated_residual_norm(xr, branch=y.to(DEV), gate=z.to(DEV)) is None                 # the sum alone
        assert torch.allclose(xr.cpu().double(), want_x + O.sigmoid(z.double()) * y.double(), rtol=1e-6, atol=2e-6)
        h = gated_residual_norm(xr, weight=w.to(DEV), eps=1e-5, out_dtype=torch.bfloat16)      # the norm alone
        assert torch.allclose(h.float().cpu().double(), O.rms_unit(xr.cpu(), 1e-5) * w.double(), rtol=1e-2, atol=1e-2)


def test_blend_of_two_normed_branches_and_logit_cap():
    from compactor_vllm import _native as N
    from compactor_vllm.layers.layernorm import dual_norm_blend
    from oracle import nununex as O

    g = torch.Generator().manual_seed(2)
    a, b = 5 * torch.randn(9, 70, generator=g), 0.01 * torch.randn(9, 70, generator=g)       # very unequal sizes
    wa, wb = 1 + 0.3 * torch.randn(70, generator=g), 1 + 0.3 * torch.randn(70, generator=g)
    got = dual_norm_blend(a.to(DEV), wa.to(DEV), b.to(DEV), wb.to(DEV), 1e-6, 0.5)
    want = 0.5 * (O.rms_unit(a, 1e-6) * wa.double() + O.rms_unit(b, 1e-6) * wb.double())
    assert torch.allclose(got.cpu().double(), want, rtol=1e-5, atol=1e-5)
    x = (40 * torch.randn(5, 33, generator=g)).to(DEV)
    out = torch.empty_like(x)
    N.check(N.lib().cvllm_softcap(N.ptr(x), x.stride(0), N.ptr(out), out.stride(0), 5, 33, 7.5, N.CVLLM_F32,
                                  N.stream(DEV)), "cvllm_softcap")
    assert torch.allclose(out.cpu().double(), 7.5 * torch.tanh(x.cpu().double() / 7.5), rtol=1e-5, atol=1e-5)
    assert out.abs().max().item() <= 7.5


@pytest.mark.parametrize("portions", [True, False])
@pytest.mark.parametrize("top,shared", [(1, 20), (3, 0), (5, 8)])
def test_routed_experts_with_weights_on_their_inputs(portions, top, shared):
    """Sigmoid scores, the `top` largest chosen, the score on the expert's INPUT (it passes the gate's nonlinearity, so
    a weight on the output gives other numbers), the shared expert behind its own gate; both the grouped path of
    portions and the per-pair path of small steps."""
    from compactor_vllm.layers.moe import ACT_SILU, ROUTE_SIGMOID, RoutedExperts
    from compactor_vllm.utils.context import reset_context, set_context
    from oracle import nununex as O

    W, E, ff, T = 24, 5, 12, 11 if portions else 3
    g = torch.Generator().manual_seed(3)
    m = RoutedExperts(W, ff, E, 0, top, 1, 1, shared, ACT_SILU, torch.float32, route_mode=ROUTE_SIGMOID,
                      shared_gate=bool(shared), scale_inputs=True).to(DEV)
    t = {"router": 1.5 * torch.randn(E, W, generator=g)}
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"] = torch.randn(ff, W, generator=g) * 0.3, torch.randn(ff, W, generator=g) * 0.3
        t[f"e{e}.down"] = torch.randn(W, ff, generator=g) * 0.3
    if shared:
        t["shared.gate"], t["shared.up"] = torch.randn(shared, W, generator=g) * 0.3, torch.randn(shared, W, generator=g) * 0.3
        t["shared.down"], t["shared.sg"] = torch.randn(W, shared, generator=g) * 0.3, torch.randn(1, W, generator=g)
    with torch.no_grad():
        m.router[:E].copy_(t["router"])
        for e in range(E):
            m.gate_up[e].copy_(torch.cat([t[f"e{e}.gate"], t[f"e{e}.up"]]))
            m.down[e].copy_(t[f"e{e}.down"])
        if shared:
            m.shared.gate_up_proj.weight.copy_(torch.cat([t["shared.gate"], t["shared.up"]]))
            m.shared.down_proj.weight.copy_(t["shared.down"])
            m.router[E:].copy_(t["shared.sg"])
    h = torch.randn(T, W, generator=g)
    f = {"router": {"experts": E, "top": top}, "shared": {"ff": shared} if shared else None}
    want = O.moe_ff(h, f, t, "")
    set_context(is_prefill=portions)
    with torch.no_grad():
        got = m(h.to(DEV))
    reset_context()
    assert torch.allclose(got.cpu().double(), want, rtol=2e-5, atol=2e-5)
    on_output = sum(O.sigmoid(O.linear(h, t["router"]))[:, e:e + 1] * O.gated_expert(h, t, f"e{e}.") for e in range(E))
    assert (want - on_output).abs().max() > 1e-3      # the case tells input weights from output weights


MIXER_CASES = {
    "delta": (gdelta(3, 12), None),
    "delta_with_moe": (gdelta(2, 16), moe(5, 2, 12, 20)),
    "parallel": (par(4, 2, 12, 10, window=7, bias_max=24, rows=8), None),
    "parallel_no_window": (par(2, 2, 16, 16, window=0, bias_max=20, rows=10), dense(24)),
    "parallel_window_of_one": (par(3, 1, 10, 6, window=1, bias_max=9, rows=4, mheads=1, mdim=4, mvdim=4), None),
    "scan": (scan(24, 6, 3, 3), None),
    "scan_without_conv": (scan(20, 16, 1, 1), dense(20)),
    "scan_wide_state": (scan(12, 40, 5, 5), None),
}


@pytest.mark.parametrize("name", sorted(MIXER_CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mixer_alone(name, dtype):
    """One layer: whole prompt, portions down to two and one tokens, token-by-token decoding."""
    from oracle import nununex as O

    r, cfg, t = build(model_cfg([MIXER_CASES[name]]), dtype, pages=12, page_size=16)
    toks = tokens(45, 83, 5)
    want = O.forward(cfg, t, toks)
    for sizes in ([45], [2], [1], [7, 1, 16, 3]):
        assert close(run_in_portions(r, toks, sizes), want, dtype), sizes


@pytest.mark.parametrize("taps", [1, 2, 5])
def test_input_convolution_of_other_lengths(taps):
    """The convolution in front of every sublayer: one tap (no history), two, and more than the fast kernels serve;
    its history crosses every cut, and a sequence's first tokens see zeros."""
    from oracle import nununex as O

    r, cfg, t = build(model_cfg([(gdelta(2, 8), dense(16)), (scan(16, 4, 2, 2), None)], taps=taps), "float32", pages=8)
    toks = tokens(30, 83, 6)
    want = O.forward(cfg, t, toks)
    for sizes in ([30], [1], [2], [3, 1, 9]):
        assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], sizes


def test_distance_buckets_match_the_oracle():
    from compactor_vllm.layers.attention import distance_buckets
    from oracle import nununex as O

    for rows, far in ((16, 120), (8, 24), (6, 12), (32, 1000), (2, 5)):
        assert distance_buckets(rows, far, far + 40) == [O.distance_bucket(n, rows, far) for n in range(far + 40)]


# ------------------------------------------------------------------------------------ window, buckets, sink: the edges
@pytest.mark.parametrize("window", [2, 5, 16, 17, 33])
def test_window_edges_in_portions_and_decoding(window):
    """The key at distance window - 1 carries a large learned bias, so it dominates every query's softmax: a window one
    token short or long changes the logits by far more than the tolerance (the oracle is asked both ways first).
    Windows shorter than, equal to and longer than a page of 16, cuts before, at and after the edge."""
    from oracle import nununex as O

    rows = 8
    cfg0 = model_cfg([(par(2, 1, 16, 16, window=window, bias_max=max(window, 9), rows=rows, mheads=1, mdim=4, mvdim=4), None)])
    r, cfg, t = build(cfg0, "float32", pages=12, page_size=16)
    rel = t["l0.mix.left.rel"].clone()
    rel[O.distance_bucket(window - 1, rows, max(window, 9))] += 6.0
    t["l0.mix.left.rel"] = rel
    r.model.load_weights(t)
    toks = tokens(80, 83, 7)
    want = O.forward(cfg, t, toks)
    for other in (window - 1, window + 1):
        alt = model_cfg([(par(2, 1, 16, 16, window=other, bias_max=max(window, 9), rows=rows, mheads=1, mdim=4, mvdim=4), None)])
        from nununex_common import clean
        assert rel_err(O.forward(clean(alt), t, toks), want) > 1e-2
    for sizes in ([80], [window, 1], [window - 1 or 1, 2], [16], [3, 64]):
        assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], sizes
    seq = new_seq()
    out = [feed(r, seq, toks[:3])] + [feed(r, seq, [x]) for x in toks[3:]]
    r.release([seq])
    assert rel_err(torch.cat(out), want) < TOL["float32"]


def test_every_bucket_of_the_distance_bias_counts():
    """No window: keys hundreds of tokens back are seen through the last buckets.  Raising one row of the table at a
    time must move the logits (oracle) and the engine must follow, in portions and decoding."""
    from oracle import nununex as O

    cfg0 = model_cfg([(par(2, 2, 16, 8, window=0, bias_max=60, rows=8, mheads=1, mdim=4, mvdim=4), None)])
    r, cfg, t = build(cfg0, "float32", pages=14, page_size=16)
    toks = tokens(200, 83, 8)
    base = O.forward(cfg, t, toks)
    for row in (0, 3, 5, 7):
        t2 = dict(t)
        rel = t["l0.mix.left.rel"].clone()
        rel[row] += 4.0
        t2["l0.mix.left.rel"] = rel
        r.model.load_weights(t2)
        want = O.forward(cfg, t2, toks)
        assert rel_err(want, base) > 1e-3
        for sizes in ([200], [150, 1, 1, 7]):
            assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], (row, sizes)


def test_a_large_sink_takes_the_weight():
    from oracle import nununex as O

    r, cfg, t = build(model_cfg([(par(2, 1, 16, 16, window=9, bias_max=20, rows=6), None)]), "float32", pages=8)
    toks = tokens(40, 83, 6)
    outs = []
    for value in (-30.0, 0.0, 9.0):
        t["l0.mix.left.sink"] = torch.tensor([value, value / 2]).to(torch.bfloat16)
        r.model.load_weights(t)
        want = O.forward(cfg, t, toks)
        outs.append(want)
        for sizes in ([40], [33, 1], [5]):
            assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], (value, sizes)
    assert (outs[0] - outs[1]).abs().max() > 1e-3 and (outs[1] - outs[2]).abs().max() > 1e-3


# ------------------------------------------------------------------- whole prompts, portions, decoding, first tokens
@pytest.mark.parametrize("dtype,cfg", [("float32", config_a), ("float32", config_b), ("bfloat16", config_b),
                                       ("bfloat16", config_a)])
def test_prefill_portions_and_decoding_agree_with_the_oracle(dtype, cfg):
    from oracle import nununex as O

    r, c, t = build(cfg(), dtype, pages=16, page_size=16)
    toks = tokens(70, c["vocab"], 7)
    want = O.forward(c, t, toks)
    for sizes in ([70], [2], [16], [17, 1, 1, 30], [3, 64]):
        assert close(run_in_portions(r, toks, sizes), want, dtype), sizes
    seq = new_seq()
    out = [feed(r, seq, toks[:1])] + [feed(r, seq, [x]) for x in toks[1:]]
    r.release([seq])
    assert close(torch.cat(out), want, dtype)


def test_residual_stream_after_every_layer():
    from oracle import nununex as O

    r, c, t = build(config_a(), "float32", pages=8)
    toks = tokens(20, 83, 8)
    want = []
    O.forward(c, t, toks, want)
    r.model.debug_residuals = got = []
    seq = new_seq()
    feed(r, seq, toks)
    r.model.debug_residuals = None
    r.release([seq])
    assert len(got) == len(want) == 6
    for i, (g, w) in enumerate(zip(got, want)):
        assert torch.allclose(g.cpu().double(), w, rtol=1e-4, atol=1e-4), i


@pytest.mark.parametrize("eager", [True, False])
def test_first_tokens_of_a_sequence(eager):
    """One-token requests, and the first steps of a request one token at a time (the graph's first replay included):
    the pair table's extra row, zeros in front of every convolution, a running maximum that starts at 0."""
    from oracle import nununex as O

    r, c, t = build(config_a(), "float32", pages=8, eager=eager)
    for seed in (1, 2):
        toks = tokens(4, 83, seed)
        want = O.forward(c, t, toks)
        seq = new_seq()
        out = [feed(r, seq, [x]) for x in toks]
        r.release([seq])
        assert rel_err(torch.cat(out), want) < TOL["float32"]
        assert rel_err(run_in_portions(r, toks[:1], [1]), want[:1]) < TOL["float32"]


@pytest.mark.parametrize("eager", [True, False])
def test_long_decoding_over_pages(eager):
    """A short prompt, then 150 single-token steps over ten pages and several windows (eager kernels, graph replays)."""
    from oracle import nununex as O

    r, c, t = build(config_a(), "float32", pages=12, eager=eager)
    toks = tokens(160, 83, 11)
    want = O.forward(c, t, toks)
    seq = new_seq()
    out = [feed(r, seq, toks[:10])] + [feed(r, seq, [x]) for x in toks[10:]]
    r.release([seq])
    if not eager:
        assert r.stats["graph_replays"] == 150
    assert rel_err(torch.cat(out), want) < TOL["float32"]


def test_graph_decode_batches_with_padding_rows():
    """Three decoding requests (padded to four rows in the graph) of unequal lengths, one of which ends early."""
    from oracle import nununex as O

    r, c, t = build(config_a(), "float32", pages=20, eager=False)
    reqs = [tokens(n, 83, 40 + i) for i, n in enumerate((30, 12, 21))]
    want = [O.forward(c, t, q) for q in reqs]
    seqs = [new_seq() for _ in reqs]
    got = [[feed(r, s, q[:4])] for s, q in zip(seqs, reqs)]
    for k in range(4, 30):
        live = [i for i, q in enumerate(reqs) if k < len(q)]
        for i in live:
            seqs[i].prompt_token_ids.append(reqs[i][k])
        logits = r.run_step([(seqs[i], [reqs[i][k]]) for i in live])
        for j, i in enumerate(live):
            got[i].append(logits[j:j + 1])
        r.release([seqs[i] for i in live if k == len(reqs[i]) - 1])
    for i in range(3):
        assert rel_err(torch.cat(got[i]), want[i]) < TOL["float32"]


# -------------------------------------------------------------------------------------------- states that must last
@pytest.mark.parametrize("kind", ["delta", "memory", "scan"])
def test_state_far_back_reaches_the_last_token(kind):
    """A recurrent layer with almost no decay: the first token is still in the state 200 tokens later, through portions
    and decoding; swapping the first token must change the last logits in the oracle, and the engine must agree."""
    from oracle import nununex as O

    if kind == "delta":      # a wide key space: the rule also erases along every new key
        layer = (gdelta(2, 64), None)
    elif kind == "memory":   # a window of one leaves the attention side without memory
        layer = (par(1, 1, 4, 4, window=1, bias_max=5, rows=4, mheads=2, mdim=8, mvdim=12, cap=6.0), None)
    else:
        layer = (scan(16, 8, 2, 2), None)
    r, cfg, t = build(model_cfg([layer], taps=1), "float32", pages=20)
    if kind == "delta":
        t["l0.mix.w0"] = torch.full_like(t["l0.mix.w0"], -14.0)
        t["l0.mix.a.b"] = torch.full_like(t["l0.mix.a.b"], -6.0)
    elif kind == "memory":
        t["l0.mix.right.f.b"] = torch.full_like(t["l0.mix.right.f.b"], 30.0)
        t["l0.mix.right.i.b"] = torch.full_like(t["l0.mix.right.i.b"], -1.0)
    else:
        t["l0.mix.A_log"] = torch.full_like(t["l0.mix.A_log"], -9.0)
    r.model.load_weights(t)
    toks = tokens(200, 83, 17)
    want = O.forward(cfg, t, toks)
    alt = [(toks[0] + 1) % 83] + toks[1:]
    assert (O.forward(cfg, t, alt)[-1] - want[-1]).abs().max().item() > 1e-3
    for sizes in ([200], [2], [16, 1, 33], [199, 1]):
        assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], sizes


def test_gates_far_beyond_the_cap():
    """Gate logits of +-60 are cut to +-cap by the tanh; the running maximum keeps every exponential in range."""
    from oracle import nununex as O

    layer = (par(1, 1, 4, 4, window=3, bias_max=5, rows=4, mheads=2, mdim=8, mvdim=12, cap=4.0), None)
    r, cfg, t = build(model_cfg([layer]), "float32", pages=8)
    t["l0.mix.right.i.b"] = torch.tensor([60.0, -60.0]).to(torch.bfloat16)
    t["l0.mix.right.f.b"] = torch.tensor([-60.0, 60.0]).to(torch.bfloat16)
    r.model.load_weights(t)
    toks = tokens(50, 83, 18)
    want = O.forward(cfg, t, toks)
    assert torch.isfinite(want).all()
    for sizes in ([50], [1], [7, 2]):
        assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], sizes


@pytest.mark.parametrize("layout", [108, 208, 216, 416, 432, 832])
def test_recurrent_layouts_give_the_same_numbers(layout):
    """The matrix-state kernels spread a head's value columns over a cluster of 1 to 8 CTAs and its key rows over
    register slices of 8 to 32 numbers; whatever the layout, the logits are the oracle's (portions and decoding)."""
    from compactor_vllm import _native as N
    from oracle import nununex as O

    cfg0 = model_cfg([(gdelta(2, 64), None), (par(1, 1, 8, 8, window=4, bias_max=9, rows=4, mheads=2, mdim=48, mvdim=64), dense(24))],
                     width=40)
    r, cfg, t = build(cfg0, "float32", pages=12)
    toks = tokens(90, 83, 12)
    want = O.forward(cfg, t, toks)
    N.set_test_option("recur_layout", layout)
    try:
        for sizes in ([90], [70, 1, 1, 3], [33]):
            assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], sizes
    finally:
        N.set_test_option("recur_layout", 0)


# ---------------------------------------------------------------------------------- batches, pages and slots reused
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_equal_each_request_alone(dtype):
    """Four requests of unequal lengths in one step after another: portions of some beside single tokens of others."""
    from oracle import nununex as O

    r, c, t = build(config_a() if dtype == "float32" else config_b(), dtype, pages=30)
    reqs = [tokens(n, c["vocab"], 70 + i) for i, n in enumerate((61, 9, 33, 2))]
    plan = [[5, 1, 1, 1, 20, 1, 1, 30, 1], [9], [1, 1, 16, 2, 13], [1, 1]]      # portion sizes per request, step by step
    seqs, at, outs = [new_seq() for _ in reqs], [0] * 4, [[] for _ in reqs]
    step = 0
    while any(at[i] < len(reqs[i]) for i in range(4)):
        entries, spans, base = [], [], 0
        for i in range(4):
            if step < len(plan[i]) and at[i] < len(reqs[i]):
                n = min(plan[i][step], len(reqs[i]) - at[i])
                part = reqs[i][at[i]:at[i] + n]
                seqs[i].prompt_token_ids.extend(part)
                entries.append((seqs[i], part))
                spans.append((i, base, n))
                at[i] += n
                base += n
        logits = r.run_step(entries, rows=list(range(base)))
        for i, b, n in spans:
            outs[i].append(logits[b:b + n])
        step += 1
    for i in range(4):
        assert close(torch.cat(outs[i]), O.forward(c, t, reqs[i]), dtype), i


@pytest.mark.parametrize("device_allocator", [False, True])
def test_pages_and_slots_are_reused(device_allocator):
    """A pool of 8 pages and 2 slots serves 6 requests, two at a time: every page and state slot is used again by a later
    request - also by a shorter one, whose first tokens must not see what the slot held before."""
    from oracle import nununex as O

    r, c, t = build(config_a(), "float32", pages=8, max_seqs=2, device_allocator=device_allocator)
    lens = (50, 60, 64, 3, 1, 49)
    for k in range(0, len(lens), 2):
        pair = [tokens(lens[k], 83, 20 + k), tokens(lens[k + 1], 83, 21 + k)]
        seqs, outs, at = [new_seq(), new_seq()], [[], []], [0, 0]
        while any(at[i] < len(pair[i]) for i in range(2)):
            entries, spans, base = [], [], 0
            for i in range(2):
                n = min(11 + 6 * i, len(pair[i]) - at[i])
                if n:
                    part = pair[i][at[i]:at[i] + n]
                    seqs[i].prompt_token_ids.extend(part)
                    entries.append((seqs[i], part))
                    spans.append((i, base, n))
                    at[i] += n
                    base += n
            logits = r.run_step(entries, rows=list(range(base)))
            for i, b, n in spans:
                outs[i].append(logits[b:b + n])
        r.release(seqs)
        for i in range(2):
            assert rel_err(torch.cat(outs[i]), O.forward(c, t, pair[i])) < TOL["float32"], (k, i)
    assert r.kv.num_free_batches == 2


def test_a_request_left_out_of_steps_goes_on_later():
    from oracle import nununex as O

    r, c, t = build(config_a(), "float32", pages=12)
    a, b = tokens(40, 83, 31), tokens(30, 83, 32)
    sa, sb = new_seq(), new_seq()
    out_a = [feed(r, sa, a[:13])]
    out_b = [feed(r, sb, b[:20]), feed(r, sb, b[20:21]), feed(r, sb, b[21:])]     # a waits meanwhile
    out_a += [feed(r, sa, a[13:14]), feed(r, sa, a[14:])]
    r.release([sa, sb])
    assert rel_err(torch.cat(out_a), O.forward(c, t, a)) < TOL["float32"]
    assert rel_err(torch.cat(out_b), O.forward(c, t, b)) < TOL["float32"]


# ------------------------------------------------------------------------------------------------------ other sizes
OTHER_SIZES = {
    "everything_one": [(par(1, 1, 1, 1, window=1, bias_max=2, rows=2, mheads=1, mdim=1, mvdim=1, cap=1.0), dense(1)),
                       (gdelta(1, 1), moe(1, 1, 1, 1)), (scan(1, 1, 1, 1), None)],
    "one_head_per_group": [(par(5, 5, 8, 8, window=6, bias_max=30, rows=8, mheads=5, mdim=8, mvdim=8), None),
                           (gdelta(3, 8), dense(16))],
    "all_heads_share_one": [(par(6, 1, 16, 8, window=12, bias_max=16, rows=6, mheads=1, mdim=16, mvdim=8), dense(32)),
                            (gdelta(6, 10), None)],
    "wide_heads": [(par(2, 1, 128, 128, window=30, bias_max=90, rows=16, mheads=2, mdim=128, mvdim=64), None),
                   (gdelta(2, 128), None), (scan(256, 16, 8, 4), dense(32))],
    "key_of_72_value_of_136": [(par(2, 2, 72, 136, window=25, bias_max=40, rows=10, mheads=1, mdim=72, mvdim=136), None),
                               (gdelta(1, 136), None)],
    "all_experts_chosen": [(gdelta(2, 8), moe(3, 3, 8, 0)), (scan(24, 20, 6, 3), moe(7, 1, 8, 40))],
    "recurrent_only": [(scan(32, 16, 4, 4), dense(32)), (gdelta(2, 16), dense(32))],
}


@pytest.mark.parametrize("name", sorted(OTHER_SIZES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(name, dtype):
    from oracle import nununex as O

    one = name == "everything_one"
    width = {"everything_one": 6, "wide_heads": 128}.get(name, 40)
    cfg0 = model_cfg(OTHER_SIZES[name], vocab=37, width=width, eps=3e-6, taps=1 if one else 4, cap=0.9 if one else 50.0,
                     buckets=1 if one else 53, mul_prev=1 if one else 11, decay_rank=1 if one else 7)
    r, cfg, t = build(cfg0, dtype, pages=10)
    toks = tokens(50, 37, 9)
    want = O.forward(cfg, t, toks)
    for sizes in ([50], [9, 2, 1]):
        assert close(run_in_portions(r, toks, sizes), want, dtype), sizes
    seq = new_seq()
    out = [feed(r, seq, toks[:31])] + [feed(r, seq, [x]) for x in toks[31:]]
    r.release([seq])
    assert close(torch.cat(out), want, dtype)


def _random_config(seed):
    g = torch.Generator().manual_seed(1000 + seed)
    ri = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    layers = []
    for _ in range(ri(2, 5)):
        kind = ri(0, 2)
        if kind == 0:
            mixer = gdelta(ri(1, 4), ri(3, 24))
        elif kind == 1:
            G = ri(1, 3)
            rows = 2 * ri(1, 8)
            mixer = par(G * ri(1, 3), G, ri(2, 24), ri(2, 24), window=ri(0, 40), bias_max=rows // 2 + ri(1, 60), rows=rows,
                        scale=0.1 + 0.05 * ri(0, 8), mheads=ri(1, 4), mdim=ri(2, 20), mvdim=ri(2, 20), cap=float(ri(2, 20)))
        else:
            mixer = scan(ri(4, 40), ri(1, 20), ri(1, 6), ri(1, 5))
        ff = ri(0, 2)
        E = ri(1, 7)
        mlp = None if ff == 0 else dense(ri(4, 50)) if ff == 1 else moe(E, ri(1, E), ri(2, 20), ri(0, 1) * ri(2, 24))
        layers.append((mixer, mlp))
    return model_cfg(layers, vocab=ri(20, 120), width=ri(8, 70), eps=10.0 ** -ri(4, 7), taps=ri(1, 5),
                     cap=float(ri(5, 40)), buckets=ri(2, 300), mul_prev=ri(1, 100000), mul_cur=ri(1, 1000),
                     decay_rank=ri(1, 9))


@pytest.mark.parametrize("seed", range(10))
def test_models_drawn_at_random(seed):
    """Layer order, every size and every constant drawn at random; whole, in portions, decoding, two in a batch."""
    from oracle import nununex as O

    cfg0 = _random_config(seed)
    r, cfg, t = build(cfg0, "float32", seed=seed, pages=16, max_seqs=2)
    a, b = tokens(57, cfg["vocab"], seed), tokens(23, cfg["vocab"], seed + 50)
    wa, wb = O.forward(cfg, t, a), O.forward(cfg, t, b)
    for sizes in ([57], [5, 1, 2, 30]):
        assert rel_err(run_in_portions(r, a, sizes), wa) < TOL["float32"], sizes
    sa, sb = new_seq(), new_seq()
    oa, ob = [feed(r, sa, a[:40])], []
    for k in range(17):
        sa.prompt_token_ids.append(a[40 + k])
        part = b[:7] if k == 0 else b[6 + k:7 + k]
        sb.prompt_token_ids.extend(part)
        logits = r.run_step([(sa, [a[40 + k]]), (sb, part)], rows=list(range(1 + len(part))))
        oa.append(logits[:1])
        ob.append(logits[1:])
    r.release([sa, sb])
    assert rel_err(torch.cat(oa), wa) < TOL["float32"]
    assert rel_err(torch.cat(ob), wb) < TOL["float32"]


# ----------------------------------------------------------------------------------------- the engine's entry point
@pytest.mark.parametrize("eager", [True, False])
def test_greedy_generation_through_llm_generate(eager):
    """`LLM.generate` with the step scheduler: prompts in portions of at most 16 tokens beside decoding requests, five
    requests on three slots, single-token steps from the decode graph.  Teacher forcing against the oracle: every
    generated token must be the oracle's argmax unless the oracle's two best logits are closer than rounding."""
    from compactor_vllm import LLM
    from compactor_vllm.api_types import SamplingParams
    from compactor_vllm.config.engine_config import LLMConfig
    from compactor_vllm.config.model_config import NununexConfig
    from nununex_common import clean, random_checkpoint
    from oracle import nununex as O

    cfg0 = config_a()
    t, c = random_checkpoint(cfg0, 3), clean(cfg0)
    cfg = LLMConfig(model="synthetic", hf_config=NununexConfig.from_json(c), dtype="float32", max_num_seqs=3,
                    kvcache_page_size=16, max_model_len=160, enforce_eager=eager)
    llm = LLM(cfg, num_pages=14, device_allocator=False, max_batched_tokens=16)
    llm.model_runner.model.load_weights(t)
    prompts = [tokens(n, 83, 30 + i) for i, n in enumerate((40, 3, 25, 1, 18))]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12))
    assert llm.model_runner.kv.num_free_batches == 3
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        logits = O.forward(c, t, p + o[:-1])[len(p) - 1:]
        for k, tok in enumerate(o):
            best = torch.topk(logits[k], 2)
            assert tok == int(best.indices[0]) or float(best.values[0] - best.values[1]) < 1e-3, (k, tok)
