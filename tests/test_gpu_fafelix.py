"""Fafelix through the engine against the plain CPU oracle (oracle/fafelix.py).

Every test makes its own small configuration and random weights.  The engine runs them through its runner
(`ModelRunner.run_step`, the paged cache, the state pool, the native kernels); the oracle recomputes whole sequences
without a cache or a carried state.  float32 runs are compared sharply (they show a key that is one position off, a
lost state or a missing sink), bfloat16 runs loosely."""
import pytest
import torch

from fafelix_common import (TOL, attn, config_a, config_b, delta, dense, feed, make_runner, model_cfg, new_seq,
                            oracle_model, rel_err, row_errs, run_in_portions, tokens, wkv)

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


def close(got, want, dtype):
    e = row_errs(got, want).flatten()
    if dtype == "float32":
        return bool(e.max() < TOL[dtype])
    return bool(e.median() < 0.03 and e.max() < 0.15)


# ------------------------------------------------------------------------------------------ mechanisms one by one
@pytest.mark.parametrize("width", [40, 257, 1024])
def test_residual_sum_and_layer_norm(width):
    from compactor_vllm.layers.layernorm import NORM_LAYER, NORM_RMS, residual_norm
    from oracle import fafelix as O

    g = torch.Generator().manual_seed(1)
    x = torch.randn(7, width, generator=g) * 3 + 1.5              # a mean far from zero: the variance needs two passes
    a = (torch.randn(7, width, generator=g) * 0.5).to(torch.bfloat16)
    b = (torch.randn(7, width, generator=g) * 0.5).to(torch.bfloat16)
    c = torch.randn(7, width, generator=g)
    w, bias = 1 + 0.2 * torch.randn(width, generator=g), 0.3 * torch.randn(width, generator=g)
    want_x = x.double() + a.double() + b.double() + c.double()
    xr = x.clone().to(DEV)
    h = residual_norm(xr, add=(a.to(DEV), b.to(DEV)), add_f32=c.to(DEV), weight=w.to(DEV), bias=bias.to(DEV), eps=1e-5,
                      kind=NORM_LAYER, out_dtype=torch.float32)
    assert torch.allclose(xr.cpu().double(), want_x, rtol=1e-6, atol=1e-6)
    assert torch.allclose(h.cpu().double(), O.layer_norm(want_x, w, bias, 1e-5), rtol=2e-5, atol=2e-5)
    h = residual_norm(xr, weight=w.to(DEV), eps=1e-5, kind=NORM_RMS, out_dtype=torch.bfloat16)   # no sum, the other norm
    assert torch.allclose(xr.cpu().double(), want_x, rtol=1e-6, atol=1e-6)
    assert torch.allclose(h.float().cpu().double(), O.rms_unit(want_x, 1e-5) * w.double(), rtol=1e-2, atol=1e-2)
    assert residual_norm(xr, add=(a.to(DEV),)) is None                                          # the sum alone
    assert torch.allclose(xr.cpu().double(), want_x + a.double(), rtol=1e-6, atol=1e-6)


def test_rotation_frequencies_in_all_three_bands():
    from compactor_vllm.layers.attention import pair_rotation_frequencies
    from oracle import fafelix as O

    for dims, base, sc in ((24, 300000.0, (6.0, 1.0, 4.0, 2048)), (64, 10000.0, (4.0, 2.0, 8.0, 512)), (8, 100.0, None),
                           (32, 500000.0, (32.0, 1.0, 4.0, 8192))):
        got, want = pair_rotation_frequencies(dims, base, sc), O.scaled_frequencies(dims, base, sc)
        assert torch.allclose(got, want, rtol=1e-12, atol=0)
        if sc:   # the case must reach kept, blended and slowed frequencies
            plain = O.scaled_frequencies(dims, base, None)
            ratio = want / plain
            assert (ratio == 1).any() and torch.isclose(ratio, torch.tensor(1 / sc[0], dtype=ratio.dtype)).any()
    blended = O.scaled_frequencies(64, 10000.0, (4.0, 2.0, 8.0, 512)) / O.scaled_frequencies(64, 10000.0, None)
    assert ((blended > 0.26) & (blended < 0.99)).any()


def test_pair_embedding_rows_across_cuts_and_slots():
    """The hashed row of a portion's first token comes from the slot's previous token; a sequence's first token takes
    the extra row whatever the slot held.  Multipliers large enough that the products need 64 bits."""
    from oracle import fafelix as O

    cfg = model_cfg([(wkv(1, 4), None)], vocab=50000, width=8, buckets=997, mul_prev=2000003, mul_cur=1000033)
    r = make_runner(cfg, "float32", pages=8, page_size=16, max_seqs=2)
    om = oracle_model(r.model)
    emb = r.model.embed
    from compactor_vllm.utils.context import reset_context, set_context

    def run(ids, pos, slots):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        set_context(is_prefill=True, positions_i32=i32(pos), token_slot=i32(slots))
        out = emb(torch.tensor(ids, dtype=torch.int64, device=DEV))
        reset_context()
        return out.cpu().double()

    toks = tokens(12, 50000, 3)
    want = O.embedding(om, toks)
    got = torch.cat([run(toks[:5], list(range(5)), [1] * 5), run(toks[5:6], [5], [1]), run(toks[6:], list(range(6, 12)), [1] * 6)])
    assert torch.allclose(got, want, rtol=0, atol=1e-6)
    # two sequences in one step, each continuing from its own slot's previous token; then a new one on a used slot
    other = tokens(7, 50000, 4)
    w2 = O.embedding(om, other)
    run(other[:3], [0, 1, 2], [2] * 3)
    both = run(other[3:5] + toks[:2], [3, 4, 0, 1], [2, 2, 1, 1])
    assert torch.allclose(both[:2], w2[3:5], atol=1e-6) and torch.allclose(both[2:], want[:2], atol=1e-6)
    assert int(emb.prev_token[1]) == toks[1] and int(emb.prev_token[2]) == other[4]


MIXER_CASES = {
    "attention": (attn(4, 2, 12, 10, 6), dense(24)),
    "attention_full_rotation": (attn(2, 2, 16, 16, 16, base=50.0, scaling=(2.0, 1.0, 2.0, 16)), None),
    "attention_no_rotation": (attn(3, 1, 10, 6, 0, scaling=None), None),
    "delta": (delta(4, 2, 12, 10, 3), None),
    "delta_with_ff": (delta(2, 1, 16, 8, 4), dense(20)),
    "wkv": (wkv(3, 12), None),
    "wkv_with_ff": (wkv(2, 20), dense(24)),
}


@pytest.mark.parametrize("name", sorted(MIXER_CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mixer_alone(name, dtype):
    """One layer: whole prompt, portions down to two and one tokens, token-by-token decoding."""
    from oracle import fafelix as O

    r = make_runner(model_cfg([MIXER_CASES[name]]), dtype, pages=12, page_size=16)
    toks = tokens(45, 83, 5)
    want = O.forward(oracle_model(r.model), toks)
    for sizes in ([45], [2], [1], [7, 1, 16, 3]):
        assert close(run_in_portions(r, toks, sizes), want, dtype), sizes


def test_a_large_sink_takes_the_weight():
    """With a sink score far above every key's score the attention output nearly vanishes; with one far below it is the
    plain softmax.  Both in the oracle and in the engine, in portions and decoding."""
    from oracle import fafelix as O

    r = make_runner(model_cfg([(attn(2, 1, 16, 16, 8), None)]), "float32", pages=8, page_size=16)
    toks = tokens(40, 83, 6)
    outs = []
    for value in (-30.0, 0.0, 9.0):
        with torch.no_grad():
            r.model.layers[0].mixer.attn.sink_logits.copy_(torch.tensor([value, value / 2]))
        want = O.forward(oracle_model(r.model), toks)
        outs.append(want)
        for sizes in ([40], [33, 1], [5]):
            assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], (value, sizes)
    assert (outs[0] - outs[1]).abs().max() > 1e-3 and (outs[1] - outs[2]).abs().max() > 1e-3


# ------------------------------------------------------------------- whole prompts, portions, decoding, first tokens
@pytest.mark.parametrize("dtype,cfg", [("float32", config_a), ("float32", config_b), ("bfloat16", config_b),
                                       ("bfloat16", config_a)])
def test_prefill_portions_and_decoding_agree_with_the_oracle(dtype, cfg):
    from oracle import fafelix as O

    r = make_runner(cfg(), dtype, pages=16, page_size=16)
    toks = tokens(70, r.model.config.vocab_size, 7)
    want = O.forward(oracle_model(r.model), toks)
    for sizes in ([70], [2], [16], [17, 1, 1, 30], [3, 64]):
        assert close(run_in_portions(r, toks, sizes), want, dtype), sizes
    seq = new_seq()
    out = [feed(r, seq, toks[:1])] + [feed(r, seq, [t]) for t in toks[1:]]
    r.release([seq])
    assert close(torch.cat(out), want, dtype)


def test_residual_stream_after_every_layer_run():
    from oracle import fafelix as O

    r = make_runner(config_a(), "float32", pages=8, page_size=16)
    toks = tokens(20, 83, 8)
    want = []
    O.forward(oracle_model(r.model), toks, want)
    r.model.debug_residuals = got = []
    seq = new_seq()
    feed(r, seq, toks)
    r.model.debug_residuals = None
    r.release([seq])
    assert len(got) == len(want) == 5 + 2
    for i, (g, w) in enumerate(zip(got, want)):
        assert torch.allclose(g.cpu().double(), w, rtol=1e-4, atol=1e-4), i


@pytest.mark.parametrize("eager", [True, False])
def test_first_tokens_of_a_sequence(eager):
    """One-token requests, and the first steps of a request one token at a time (the graph's first replay included)."""
    from oracle import fafelix as O

    r = make_runner(config_a(), "float32", pages=8, page_size=16, eager=eager)
    om = oracle_model(r.model)
    for seed in (1, 2):
        toks = tokens(4, 83, seed)
        want = O.forward(om, toks)
        seq = new_seq()
        out = [feed(r, seq, [t]) for t in toks]
        r.release([seq])
        assert rel_err(torch.cat(out), want) < TOL["float32"]
        assert rel_err(run_in_portions(r, toks[:1], [1]), want[:1]) < TOL["float32"]


@pytest.mark.parametrize("eager", [True, False])
def test_long_decoding_over_pages(eager):
    """A short prompt, then 150 single-token steps over ten pages (eager kernels, and replays of the decode graph)."""
    from oracle import fafelix as O

    r = make_runner(config_a(), "float32", pages=12, page_size=16, eager=eager)
    toks = tokens(160, 83, 11)
    want = O.forward(oracle_model(r.model), toks)
    seq = new_seq()
    out = [feed(r, seq, toks[:10])] + [feed(r, seq, [t]) for t in toks[10:]]
    r.release([seq])
    if not eager:
        assert r.stats["graph_replays"] == 150
    assert rel_err(torch.cat(out), want) < TOL["float32"]


def test_graph_decode_batches_with_padding_rows():
    """Three decoding requests (padded to four rows in the graph) of unequal lengths, one of which ends early."""
    from oracle import fafelix as O

    r = make_runner(config_a(), "float32", pages=20, page_size=16, eager=False)
    om = oracle_model(r.model)
    reqs = [tokens(n, 83, 40 + i) for i, n in enumerate((30, 12, 21))]
    want = [O.forward(om, t) for t in reqs]
    seqs = [new_seq() for _ in reqs]
    got = [[feed(r, s, t[:4])] for s, t in zip(seqs, reqs)]
    for k in range(4, 30):
        live = [i for i, t in enumerate(reqs) if k < len(t)]
        for i in live:
            seqs[i].prompt_token_ids.append(reqs[i][k])
        logits = r.run_step([(seqs[i], [reqs[i][k]]) for i in live])
        for j, i in enumerate(live):
            got[i].append(logits[j:j + 1])
        r.release([seqs[i] for i in live if k == len(reqs[i]) - 1])
    for i in range(3):
        assert rel_err(torch.cat(got[i]), want[i]) < TOL["float32"]


# ------------------------------------------------------------------------------ a key that stands out, far and at edges
def _standout(far, query, n, page_size=16):
    """One attention layer whose weights make ONE key stand out for one query: token 1 sits at `far`, token 2 at `query`,
    token 0 everywhere else; head 0's query of the token at `query` is turned onto the key at `far` (their rotated
    parts are small: 4 of 32 numbers)."""
    from oracle import fafelix as O

    r = make_runner(model_cfg([(attn(2, 1, 32, 16, 4, base=20.0, scaling=None, scale=1.0), None)]), "float32", pages=40,
                    page_size=page_size)
    toks = [0] * n
    toks[far], toks[query] = 1, 2
    om = oracle_model(r.model)
    L = om["layers"][0]
    h = O.layer_norm(O.embedding(om, toks), L["norm1"], L["norm1_b"], om["eps"])
    m = L["mixer"]
    k_far = h[far] @ m["k"].double().T + m["k_b"].double()                 # the one kv head's key before rotation
    hq = h[query]
    wq = m["q"].double().clone()
    cur = wq[:32] @ hq + m["q_b"].double()[:32]
    wq[:32] += torch.outer(3.0 * k_far - cur, hq) / (hq @ hq)
    layer = r.model.layers[0]
    with torch.no_grad():
        layer.in_proj.weight[:64].copy_(wq.to(layer.in_proj.weight.dtype))
    return r, toks


@pytest.mark.parametrize("far,query", [(0, 255), (3, 250), (15, 16), (16, 17), (31, 32), (15, 31), (16, 300), (63, 64)])
def test_standout_key_far_away_and_at_page_borders(far, query):
    from oracle import fafelix as O

    n = query + 2
    r, toks = _standout(far, query, n)
    om = oracle_model(r.model)
    want = O.forward(om, toks)
    alt = list(toks)
    alt[far] = 0         # the oracle itself must react to the far key, else the case shows nothing
    assert (O.forward(om, alt)[query] - want[query]).abs().max().item() > 1e-2
    for sizes in ([n], [50, 29], [query, 1, 1], [far + 1, 7]):
        assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], sizes
    seq = new_seq()
    out = [feed(r, seq, toks[:far + 1])] + [feed(r, seq, [t]) for t in toks[far + 1:]]
    r.release([seq])
    assert rel_err(torch.cat(out), want) < TOL["float32"]


@pytest.mark.parametrize("kind", ["delta", "wkv"])
def test_state_far_back_reaches_the_last_token(kind):
    """A recurrent layer with almost no decay: the first token is still in the state 200 tokens later, through portions
    and decoding; swapping the first token must change the last logits in the oracle and the engine alike."""
    from oracle import fafelix as O

    # the delta rule also erases along every new key: a key space of 64 keeps the first token through 200 updates
    r = make_runner(model_cfg([(delta(2, 1, 64, 12, 4) if kind == "delta" else wkv(2, 8), None)]), "float32", pages=20,
                    page_size=16)
    mx = r.model.layers[0].mixer
    with torch.no_grad():
        if kind == "delta":
            mx.A_log.fill_(-12.0)
        else:
            mx.w0.fill_(-12.0)
    om = oracle_model(r.model)
    toks = tokens(200, 83, 17)
    want = O.forward(om, toks)
    alt = [(toks[0] + 1) % 83] + toks[1:]
    assert (O.forward(om, alt)[-1] - want[-1]).abs().max().item() > 1e-3
    for sizes in ([200], [2], [16, 1, 33], [199, 1]):
        assert rel_err(run_in_portions(r, toks, sizes), want) < TOL["float32"], sizes


@pytest.mark.parametrize("layout", [108, 208, 216, 416, 432, 832])
def test_recurrent_layouts_give_the_same_numbers(layout):
    """The matrix-state kernels spread a head's value columns over a cluster of 1 to 8 CTAs and its key rows over
    register slices of 8 to 32 numbers; whatever the layout, the logits are the oracle's (portions and decoding)."""
    from compactor_vllm import _native as N
    from oracle import fafelix as O

    cfg = model_cfg([(delta(2, 1, 48, 64, 3), None), (wkv(2, 64), dense(24))], width=40, loop=(0, 2, 2))
    r = make_runner(cfg, "float32", pages=12, page_size=16)
    toks = tokens(90, 83, 12)
    want = O.forward(oracle_model(r.model), toks)
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
    from oracle import fafelix as O

    r = make_runner(config_a() if dtype == "float32" else config_b(), dtype, pages=30, page_size=16)
    om = oracle_model(r.model)
    reqs = [tokens(n, r.model.config.vocab_size, 70 + i) for i, n in enumerate((61, 9, 33, 2))]
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
        assert close(torch.cat(outs[i]), O.forward(om, reqs[i]), dtype), i


@pytest.mark.parametrize("device_allocator", [False, True])
def test_pages_and_slots_are_reused(device_allocator):
    """A pool of 8 pages and 2 slots serves 6 requests, two at a time: every page and state slot is used again by a later
    request - also by a shorter one, whose first tokens must not see what the slot held before."""
    from oracle import fafelix as O

    r = make_runner(config_a(), "float32", pages=8, page_size=16, max_seqs=2, device_allocator=device_allocator)
    om = oracle_model(r.model)
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
            assert rel_err(torch.cat(outs[i]), O.forward(om, pair[i])) < TOL["float32"], (k, i)
    assert r.kv.num_free_batches == 2


def test_a_request_left_out_of_steps_goes_on_later():
    from oracle import fafelix as O

    r = make_runner(config_a(), "float32", pages=12, page_size=16)
    om = oracle_model(r.model)
    a, b = tokens(40, 83, 31), tokens(30, 83, 32)
    sa, sb = new_seq(), new_seq()
    out_a = [feed(r, sa, a[:13])]
    out_b = [feed(r, sb, b[:20]), feed(r, sb, b[20:21]), feed(r, sb, b[21:])]     # a waits meanwhile
    out_a += [feed(r, sa, a[13:14]), feed(r, sa, a[14:])]
    r.release([sa, sb])
    assert rel_err(torch.cat(out_a), O.forward(om, a)) < TOL["float32"]
    assert rel_err(torch.cat(out_b), O.forward(om, b)) < TOL["float32"]


# ------------------------------------------------------------------------------------------------------ other sizes
OTHER_SIZES = {
    "everything_one": [(attn(1, 1, 2, 1, 2, scaling=None), dense(1)), (delta(1, 1, 1, 1, 2), dense(1)), (wkv(1, 1), None)],
    "one_head_per_group": [(attn(5, 5, 8, 8, 4), None), (delta(3, 3, 8, 8, 2), dense(16))],
    "all_heads_share_one": [(attn(6, 1, 16, 8, 16), dense(32)), (delta(6, 1, 10, 4, 5), None)],
    "wide_heads": [(attn(2, 1, 128, 128, 64, base=1e4), None), (delta(2, 1, 128, 64, 4), None), (wkv(2, 64), dense(32))],
    "key_of_72_value_of_136": [(attn(2, 2, 72, 136, 24), None), (delta(1, 1, 72, 136, 3), None), (wkv(1, 136), None)],
    "recurrent_only": [(wkv(2, 16), dense(32)), (delta(2, 2, 16, 16, 4), dense(32))],
    "attention_only": [(attn(4, 2, 16, 16, 8), dense(32)), (attn(2, 2, 32, 16, 32), None)],
}


@pytest.mark.parametrize("name", sorted(OTHER_SIZES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(name, dtype):
    from oracle import fafelix as O

    loop = {"recurrent_only": (0, 2, 2), "attention_only": (1, 2, 3), "wide_heads": (0, 3, 2)}.get(name)
    width = {"everything_one": 6, "wide_heads": 128}.get(name, 40)
    cfg = model_cfg(OTHER_SIZES[name], vocab=37, width=width, eps=3e-6, loop=loop,
                    buckets=1 if name == "everything_one" else 53, mul_prev=1 if name == "everything_one" else 11)
    r = make_runner(cfg, dtype, pages=10, page_size=16)
    toks = tokens(50, 37, 9)
    want = O.forward(oracle_model(r.model), toks)
    for sizes in ([50], [9, 2, 1]):
        assert close(run_in_portions(r, toks, sizes), want, dtype), sizes
    seq = new_seq()
    out = [feed(r, seq, toks[:31])] + [feed(r, seq, [t]) for t in toks[31:]]
    r.release([seq])
    assert close(torch.cat(out), want, dtype)


def _random_config(seed):
    g = torch.Generator().manual_seed(1000 + seed)
    ri = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    layers = []
    for _ in range(ri(2, 5)):
        kind = ("attention", "delta", "wkv")[ri(0, 2)]
        G = ri(1, 3)
        H = G * ri(1, 3)
        D = 2 * ri(2, 12)
        if kind == "attention":
            rot = 2 * ri(0, D // 2)
            sc = None if ri(0, 1) else (float(ri(2, 8)), 1.0, float(ri(2, 4)), 2 ** ri(3, 7))
            mixer = attn(H, G, D, ri(2, 24), rot, base=float(10 ** ri(1, 5)), scaling=sc, scale=0.5 + 0.1 * ri(0, 10))
        elif kind == "delta":
            mixer = delta(H, G, D, ri(2, 24), ri(2, 5))
        else:
            mixer = wkv(H, D)
        layers.append((mixer, dense(ri(4, 40)) if ri(0, 3) else None))
    n = len(layers)
    start = ri(0, n - 1)
    loop = None if ri(0, 2) == 0 else (start, ri(start + 1, n), ri(1, 3))
    return model_cfg(layers, vocab=ri(20, 90), width=4 * ri(4, 16), eps=10.0 ** -ri(4, 7), loop=loop, buckets=ri(2, 200),
                     mul_prev=ri(1, 5000), mul_cur=ri(1, 5000))


@pytest.mark.parametrize("seed", range(10))
def test_random_configurations(seed):
    """Models drawn at random (layer order, loop, every size and constant): whole prompt, portions, graph decoding and a
    two-request batch against the oracle."""
    from oracle import fafelix as O

    cfg = _random_config(seed)
    r = make_runner(cfg, "float32", pages=16, page_size=16, eager=False, seed=seed)
    om = oracle_model(r.model)
    V = cfg["vocab"]
    a, b = tokens(44, V, seed), tokens(19, V, seed + 100)
    wa, wb = O.forward(om, a), O.forward(om, b)
    assert rel_err(run_in_portions(r, a, [44]), wa) < TOL["float32"]
    assert rel_err(run_in_portions(r, a, [5, 2, 17]), wa) < TOL["float32"]
    sa, sb = new_seq(), new_seq()
    out_a, out_b = [feed(r, sa, a[:30])], []
    for k in range(14):
        entries = [(sa, [a[30 + k]])]
        sa.prompt_token_ids.append(a[30 + k])
        if k == 3:
            sb.prompt_token_ids.extend(b[:9])
            entries.append((sb, b[:9]))
        elif 3 < k < 14:
            sb.prompt_token_ids.append(b[9 + k - 4])
            entries.append((sb, [b[9 + k - 4]]))
        n = sum(len(t) for _, t in entries)
        logits = r.run_step(entries, rows=list(range(n)))
        out_a.append(logits[:1])
        if len(entries) > 1:
            out_b.append(logits[1:])
    r.release([sa, sb])
    assert rel_err(torch.cat(out_a), wa) < TOL["float32"]
    assert rel_err(torch.cat(out_b), wb) < TOL["float32"]


# ------------------------------------------------------------------------------ generation through the entry point
def test_greedy_generation_through_llm_generate():
    """`LLM.generate` with the step scheduler: prompts in portions of at most 16 tokens beside decoding requests, five
    requests on three slots.  Teacher forcing against the oracle: every generated token must be the oracle's argmax
    unless the oracle's two best logits are closer than the engine's rounding."""
    from compactor_vllm import LLM
    from compactor_vllm.api_types import SamplingParams
    from compactor_vllm.config.engine_config import LLMConfig
    from compactor_vllm.config.model_config import FafelixConfig
    from oracle import fafelix as O

    hf = FafelixConfig.from_json(config_a())
    cfg = LLMConfig(model="synthetic", hf_config=hf, dtype="float32", max_num_seqs=3, kvcache_page_size=16,
                    max_model_len=160)
    llm = LLM(cfg, num_pages=14, device_allocator=False, max_batched_tokens=16)
    om = oracle_model(llm.model_runner.model)
    prompts = [tokens(n, 83, 30 + i) for i, n in enumerate((40, 3, 25, 1, 18))]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12))
    assert llm.model_runner.kv.num_free_batches == 3
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        logits = O.forward(om, p + o[:-1])[len(p) - 1:]
        for k, tok in enumerate(o):
            best = torch.topk(logits[k], 2)
            assert tok == int(best.indices[0]) or float(best.values[0] - best.values[1]) < 1e-3, (k, tok)
