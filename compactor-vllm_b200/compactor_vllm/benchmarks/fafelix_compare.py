"""Prefill and decode throughput of a Fafelix model beside a Batasun and a Movolorn model of equal size (random weights),
all through the engine's runner, plus the design's kernels timed alone against the measured peaks.

Used by `bench.py --arch fafelix`; the default workload of bench.py does not touch this module.  Batasun is the closest
existing model: attention over the same paged kernels beside recurrent layers whose state lives in the state pool, the
same runner path (mixed steps, decode graphs) and a 32-bit residual stream; Movolorn with a dense feed-forward is the
closest to a Fafelix model of attention layers only.
Timing as in arch_compare: CUDA events on the launching stream after warm-up, a buffer larger than L2 written between
timed kernel iterations; engine-level numbers include the runner's host work.
"""
from __future__ import annotations

import json
from typing import List

import torch

from compactor_vllm.benchmarks.arch_compare import (DECODE_BATCH, DECODE_CONTEXT, DECODE_STEPS, HEAD_DIM, PREFILL_TOKENS,
                                                    SIZES, _events_ms, engine_throughput, movolorn_config)
from compactor_vllm.benchmarks.batasun_compare import batasun_config

DELTA_DIM, WKV_DIM, CONV = 128, 64, 4


def fafelix_config(s: dict, pattern: str, loop=None) -> dict:
    """`pattern`: one letter per layer, cycled over the size's layer count: A attention, D gated delta rule, W wkv."""
    W = s["width"]
    dense = {"kind": "dense", "ff": s["ff"]}
    layers = []
    for i in range(s["layers"]):
        kind = pattern[i % len(pattern)]
        if kind == "A":
            mixer = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": HEAD_DIM, "vdim": HEAD_DIM,
                     "scale": HEAD_DIM ** -0.5,
                     "rot": {"base": 500000.0, "dims": HEAD_DIM // 2,
                             "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
            layers.append({"type": "attention", "mixer": mixer, "mlp": dense})
        elif kind == "D":
            heads = W // DELTA_DIM
            layers.append({"type": "delta", "mlp": dense,
                           "mixer": {"heads": heads, "kv_heads": max(heads // 2, 1), "dim": DELTA_DIM, "vdim": DELTA_DIM,
                                     "conv": CONV}})
        else:
            layers.append({"type": "wkv", "mlp": dense, "mixer": {"heads": W // WKV_DIM, "dim": WKV_DIM, "decay_rank": 64}})
    c = {"architecture": "Fafelix", "vocab": s["vocab"], "width": W, "norm": {"eps": 1e-6},
         "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}}, "layers": layers}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


def kernel_rooflines(peaks: dict, reps: int) -> List[dict]:
    """The design's kernels alone at width 4096, bfloat16: achieved rate and its fraction of the measured copy
    bandwidth / cuBLAS bf16 rate."""
    from compactor_vllm import _native as N
    from compactor_vllm.config.constants import RESERVED_BATCH
    from compactor_vllm.kv_cache.page_table import KVAllocationStatus, PagedKVCache
    from compactor_vllm.layers.attention import BiasedChunkAttention, pair_rotation_frequencies
    from compactor_vllm.layers.layernorm import NORM_LAYER, residual_norm
    from compactor_vllm.layers.pair_embedding import HashedPairEmbedding
    from compactor_vllm.layers.recurrent import DeltaRuleMixer, WkvMixer
    from compactor_vllm.utils.context import reset_context, set_context

    dev = torch.device("cuda", torch.cuda.current_device())
    bf = torch.bfloat16
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hbm = float(peaks["hbm"]) * 1e9
    tflops = float(peaks["tensor_burst"]) * 1e12
    rows: List[dict] = []
    lib, code, st = N.lib(), N.CVLLM_BF16, N.stream(dev)

    def timed(fn):
        def run():
            flush_buf.zero_()
            fn()
        return max(_events_ms(run, reps) - _events_ms(lambda: flush_buf.zero_(), reps), 1e-4)

    def add(name, ms, *, nbytes=None, flops=None, like=None):
        r = {"kernel": name, "ms": round(ms, 4), "like": like}
        if nbytes is not None:
            r["GBs"] = round(nbytes / ms / 1e6, 1)
            r["frac_hbm_of_measured"] = round(nbytes / (ms * 1e-3) / hbm, 3)
        if flops is not None:
            r["TFLOPs"] = round(flops / ms / 1e9, 2)
            r["frac_bf16_of_measured"] = round(flops / (ms * 1e-3) / tflops, 4)
        rows.append(r)

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    T, W, PS, L = 8192, 4096, 128, 4096
    # --- the residual update of this design: two branches (4 B) + the residual read and written (8 B) + the normed row (2 B)
    x = torch.randn(T, W, device=dev)
    ya, yb = torch.randn(T, W, device=dev).to(bf), torch.randn(T, W, device=dev).to(bf)
    w1, b1 = torch.ones(W, device=dev), torch.zeros(W, device=dev)
    add("residual_norm (two branches, layer norm)",
        timed(lambda: residual_norm(x, add=(ya, yb), weight=w1, bias=b1, kind=NORM_LAYER, out_dtype=bf)),
        nbytes=14 * T * W, like="sandwich_norm")
    del x, ya, yb
    prev = torch.get_default_dtype()
    torch.set_default_dtype(bf)          # as the runner builds models: 16-bit matrices, fp32 gains, 64-bit frequencies
    H, G, D = 32, 8, 128
    try:
        with torch.device(dev):
            emb = HashedPairEmbedding(32000, W, 65521, 1000003, 31)
            attn = BiasedChunkAttention(H, G, D, D, D ** -0.5, sink=True, learned_sink=True, norm=True,
                                        rotation=pair_rotation_frequencies(64, 500000.0, (8.0, 1.0, 4.0, 8192)).to(dev))
            dm = DeltaRuleMixer(W, W // DELTA_DIM, W // DELTA_DIM // 2, DELTA_DIM, DELTA_DIM, CONV, 1e-6)
            wm = WkvMixer(W, W // WKV_DIM, WKV_DIM, 64, 1e-6, dtype=bf)
    finally:
        torch.set_default_dtype(prev)
    cache = PagedKVCache(1, L // PS + 1, (L // PS + 1) * 9 * G, PS, G, D, 9, bf, device=dev, v_head_dim=D)
    attn.k_cache, attn.v_cache, attn.page_table, attn.bh_seq_lens = cache.layer_slices(0)
    attn.page_size = PS
    slots = []
    for _ in range(8):
        s = cache.new_batch()
        assert cache.reserve_tokens(s, L + 1) == KVAllocationStatus.SUCCESS
        slots.append(s)
    pos_all = torch.arange(L, dtype=torch.int32, device=dev)
    tok_slot = torch.full((L,), slots[0], dtype=torch.int32, device=dev)
    set_context(is_prefill=True, cu_seqlens_q=i32([0, L]), max_seqlen_q=L, max_seqlen_k=L, batch_mapping=i32(slots[:1]),
                positions_i32=pos_all, token_slot=tok_slot, seq_start=i32([0]))
    emb.prev_token = torch.zeros(9, 1, dtype=torch.int32, device=dev)
    ids = torch.randint(0, 32000, (L,), device=dev)
    add("pair_hash_embed (4096 tokens)", timed(lambda: emb(ids)), nbytes=L * W * (2 + 2 + 4), like="embedding gather")
    # --- attention: rotation + norm + store, then the portion kernel with a learned sink
    qkv = torch.randn(L, attn.qkv_width, device=dev).to(bf)
    q = torch.empty(L, H, D, dtype=bf, device=dev)
    pt = attn.page_table
    table = (N.ptr(pt), pt.stride(0), pt.stride(1), PS)

    def store():
        N.check(lib.cvllm_rope_qknorm_store(N.ptr(qkv), qkv.stride(0), N.ptr(attn.inv_freq), 64, 1, None, None, 1e-6,
                                            N.ptr(pos_all), N.ptr(tok_slot), N.ptr(q), N.ptr(attn.k_cache),
                                            N.ptr(attn.v_cache), *table, N.ptr(attn.bh_seq_lens), L, H, G, D, D,
                                            RESERVED_BATCH, code, st), "store")

    add("rope_qknorm_store (4096 tokens)", timed(store), nbytes=2 * L * 2 * (H + 2 * G) * D, like="qknorm_store")
    add("portion attention with learned sinks (4096 tokens, 32 / 8 heads of 128; tcgen05 pipeline)",
        timed(lambda: attn.attend(q)), flops=4.0 * D * H * L * (L + 1) / 2, like="prefill_attn_bias")
    B = 8
    set_context(is_prefill=False, batch_mapping=i32(slots), positions_i32=i32([L - 1] * B), token_slot=i32(slots),
                max_seqlen_q=1, max_seqlen_k=L)
    qd = torch.randn(B, H, D, device=dev).to(bf)
    add("bias_attn_decode with learned sinks (8 x 4096 keys)", timed(lambda: attn.attend(qd)),
        nbytes=2 * 2 * B * G * L * D, like="bias_attn_decode")
    reset_context()
    # --- gated delta rule: 32 heads of 128 x 128
    cu, st0, bm1 = i32([0, L]), i32([0]), i32(slots[:1])
    pre = (N.ptr(cu), N.ptr(st0), None)
    posd, bmd = i32([L - 1] * B), i32(slots)
    dec = (None, None, N.ptr(posd))
    Hd, Gd, Cd = dm.heads, dm.kv_heads, dm.conv_channels
    cols = torch.randn(L, dm.in_cols, device=dev).to(bf)
    qkvf = torch.randn(L, Cd, device=dev)
    dstate = torch.zeros(9, Hd, DELTA_DIM, DELTA_DIM, device=dev)
    dout = torch.empty(L, Hd * DELTA_DIM, dtype=bf, device=dev)
    with torch.no_grad():
        dm.dt_bias.fill_(-1.0)

    def delta(geom, bm, Bn, mx_new):
        g_off = Cd
        b_off = Cd + Hd * DELTA_DIM
        N.check(lib.cvllm_delta_rule(N.ptr(qkvf), qkvf.stride(0), N.ptr(cols), cols.stride(0), b_off, b_off + Hd,
                                     N.ptr(dm.A_log), N.ptr(dm.dt_bias), N.ptr(dstate), N.ptr(cols), cols.stride(0),
                                     g_off, N.ptr(dm.norm_weight), 0, 1e-6, *geom, N.ptr(bm), Bn, mx_new, N.ptr(dout),
                                     dout.stride(0), Hd, Gd, DELTA_DIM, DELTA_DIM, RESERVED_BATCH, code, st), "delta")

    d_flops = 6.0 * DELTA_DIM * DELTA_DIM * Hd          # two dot products and the update per (token, head)
    add(f"delta_rule (one portion of 4096 tokens, {Hd} heads of 128 x 128, with the gated norm)",
        timed(lambda: delta(pre, bm1, 1, L)), nbytes=L * (4 * Cd + 2 * 2 * Hd * DELTA_DIM), flops=None,
        like="ssm_scan + gated_group_norm (the mixer's portion kernel)")
    rows[-1]["GFLOPs_fp32"] = round(d_flops * L / rows[-1]["ms"] / 1e6, 1)
    add("delta_rule (decode, 8 sequences: state read + written)", timed(lambda: delta(dec, bmd, B, 1)),
        nbytes=2 * 4 * B * Hd * DELTA_DIM * DELTA_DIM, like="ssm_scan (decode)")
    # --- wkv: 64 heads of 64 x 64
    Hw = wm.heads
    HD = Hw * WKV_DIM
    hin = torch.randn(L, W, device=dev).to(bf)
    shift = torch.zeros(9, W, dtype=bf, device=dev)
    blends = torch.empty(5, L, W, dtype=bf, device=dev)
    with torch.no_grad():
        wm.mu.uniform_(0, 1)
        wm.w0.fill_(-1.0)

    def tshift(geom, bm, Bn, mx_new, total):
        N.check(lib.cvllm_token_shift_mix(N.ptr(hin), hin.stride(0), N.ptr(wm.mu), 5, W, N.ptr(shift), *geom, N.ptr(bm),
                                          Bn, mx_new, N.ptr(blends), total, RESERVED_BATCH, code, st), "shift")

    add("token_shift_mix (4096 tokens, 5 blends)", timed(lambda: tshift(pre, bm1, 1, L, L)), nbytes=2 * L * W * 6,
        like="sandwich_norm")
    rk = torch.randn(4, L, HD, device=dev).to(bf)
    wraw = torch.randn(L, HD, device=dev).to(bf)
    wstate = torch.zeros(9, Hw, WKV_DIM, WKV_DIM, device=dev)
    wout = torch.empty(L, HD, dtype=bf, device=dev)

    def wkv(geom, bm, Bn, mx_new):
        N.check(lib.cvllm_wkv_scan(N.ptr(rk[0]), HD, N.ptr(rk[1]), HD, N.ptr(rk[2]), HD, N.ptr(wraw), HD, N.ptr(wm.w0),
                                   N.ptr(wm.bonus), N.ptr(wstate), N.ptr(rk[3]), HD, 0, N.ptr(wm.norm_weight), WKV_DIM,
                                   1e-6, *geom, N.ptr(bm), Bn, mx_new, N.ptr(wout), HD, Hw, WKV_DIM, RESERVED_BATCH, code,
                                   st), "wkv")

    add(f"wkv_scan (one portion of 4096 tokens, {Hw} heads of 64 x 64, with the gated norm)",
        timed(lambda: wkv(pre, bm1, 1, L)), nbytes=2 * L * HD * 6,
        like="ssm_scan + gated_group_norm (the mixer's portion kernel)")
    rows[-1]["GFLOPs_fp32"] = round(8.0 * WKV_DIM * WKV_DIM * Hw * L / rows[-1]["ms"] / 1e6, 1)
    add("wkv_scan (decode, 8 sequences: state read + written)", timed(lambda: wkv(dec, bmd, B, 1)),
        nbytes=2 * 4 * B * Hw * WKV_DIM * WKV_DIM, like="ssm_scan (decode)")
    return rows


def run(peaks: dict, sizes: List[str], reps: int) -> dict:
    from compactor_vllm.config.model_config import BatasunConfig, FafelixConfig, MovolornConfig

    result = {"arch": "fafelix", "closest": "batasun (latent attention + state-space layers); movolorn (dense) for "
                                            "attention-only models", "dtype": "bf16",
              "data": "synthetic (random weights)",
              "workload": {"prefill_tokens": PREFILL_TOKENS, "decode_batch": DECODE_BATCH,
                           "decode_context": DECODE_CONTEXT, "decode_steps": DECODE_STEPS}, "sizes": {}}
    for name in sizes:
        s = SIZES[name]
        row = {"shape": s}
        row["movolorn_dense_nochunk"] = engine_throughput("movolorn", MovolornConfig.from_json(movolorn_config(s, 0, False)), reps)
        row["batasun_mixed"] = engine_throughput("batasun", BatasunConfig.from_json(batasun_config(s, "AaMM")), reps)
        row["batasun_state_space_only"] = engine_throughput("batasun", BatasunConfig.from_json(batasun_config(s, "M")), reps)
        for label, pattern in (("fafelix_attention_only", "A"), ("fafelix_delta_only", "D"), ("fafelix_wkv_only", "W"),
                               ("fafelix_mixed", "AWDA")):
            row[label] = engine_throughput("fafelix", FafelixConfig.from_json(fafelix_config(s, pattern)), reps)
        result["sizes"][name] = row
    result["kernels"] = kernel_rooflines(peaks, max(reps, 5))
    result["peaks"] = peaks
    return result


def main(peaks: dict, sizes: str, reps: int) -> None:
    print(json.dumps(run(peaks, [x for x in sizes.split(",") if x], reps)))
