"""Prefill and decode throughput of a Nununex model beside a Fafelix and a Batasun model of equal size (random weights),
all through the engine's runner, plus the design's kernels timed alone against the measured peaks.

Used by `bench.py --arch nununex`; the default workload of bench.py does not touch this module.  Fafelix is the
closest existing model: the same hashed pair embedding, attention with learned sinks over the same paged kernels, and
matrix-state mixers on the same recurrence kernels' layout; Batasun's state-space layers stand beside the selective
scan and its routed experts beside this design's.
Timing as in arch_compare: CUDA events on the launching stream after warm-up, a buffer larger than L2 written between
timed kernel iterations; engine-level numbers include the runner's host work.
"""
from __future__ import annotations

import json
import math
from typing import List

import torch

from compactor_vllm.benchmarks.arch_compare import (DECODE_BATCH, DECODE_CONTEXT, DECODE_STEPS, HEAD_DIM, PREFILL_TOKENS,
                                                    SIZES, _events_ms, engine_throughput)
from compactor_vllm.benchmarks.batasun_compare import batasun_config
from compactor_vllm.benchmarks.fafelix_compare import fafelix_config

DELTA_DIM, MEMORY_DIM, STATE, DT_RANK, CONV, TAPS, WINDOW = 64, 128, 16, 128, 4, 4, 1024


def nununex_config(s: dict, pattern: str, moe: bool = False) -> dict:
    """`pattern`: one letter per layer, cycled over the size's layer count: G general delta rule, P windowed attention
    beside a matrix memory, S selective scan."""
    W = s["width"]
    if moe:    # 8 experts of a quarter of the dense size, 2 per token, plus a shared one: about the dense layer's work
        mlp = {"kind": "moe", "expert": {"ff": s["ff"] // 4}, "shared": {"ff": s["ff"] // 2},
               "router": {"experts": 8, "top": 2}}
    else:
        mlp = {"kind": "dense", "ff": s["ff"]}
    layers = []
    for i in range(s["layers"]):
        kind = pattern[i % len(pattern)]
        if kind == "G":
            layers.append({"type": "general_delta", "mlp": mlp, "mixer": {"heads": W // DELTA_DIM, "dim": DELTA_DIM,
                                                                          "decay_rank": 64}})
        elif kind == "P":
            left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": HEAD_DIM, "vdim": HEAD_DIM,
                    "scale": HEAD_DIM ** -0.5, "bias_max": 512, "bias_rows": 32, "mask": {"size": WINDOW}}
            right = {"heads": W // 2 // MEMORY_DIM, "dim": MEMORY_DIM, "vdim": MEMORY_DIM, "gate_cap": 15.0}
            layers.append({"type": "parallel", "mlp": mlp, "mixer": {"left": left, "right": right}})
        else:
            layers.append({"type": "mamba1", "mlp": mlp,
                           "mixer": {"inner": 2 * W, "state": STATE, "dt_rank": DT_RANK, "conv": CONV}})
    return {"architecture": "Nununex", "vocab": s["vocab"], "width": W, "norm": {"eps": 1e-6}, "canon": {"taps": TAPS},
            "logit_softcap": 30.0, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}},
            "layers": layers}


def kernel_rooflines(peaks: dict, reps: int) -> List[dict]:
    """The design's kernels alone at width 4096, bfloat16: achieved rate and its fraction of the measured copy
    bandwidth / cuBLAS bf16 rate."""
    from compactor_vllm import _native as N
    from compactor_vllm.config.constants import RESERVED_BATCH
    from compactor_vllm.kv_cache.page_table import KVAllocationStatus, PagedKVCache
    from compactor_vllm.layers.attention import BiasedChunkAttention
    from compactor_vllm.layers.layernorm import dual_norm_blend, gated_residual_norm
    from compactor_vllm.layers.recurrent import GATE_SIGMOID
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
    T, W, PS, L, B = 8192, 4096, 128, 4096, 8
    # --- the residual update: branch + gate logits (4 B) + the residual read and written (8 B) + the normed row (2 B)
    x = torch.randn(T, W, device=dev)
    y, gz = torch.randn(T, W, device=dev).to(bf), torch.randn(T, W, device=dev).to(bf)
    w1 = torch.ones(W, device=dev)
    add("gated_residual_norm (branch, gate, rms norm)",
        timed(lambda: gated_residual_norm(x, branch=y, gate=gz, weight=w1, out_dtype=bf)), nbytes=14 * T * W,
        like="residual_norm")
    add("dual_norm_blend (two branches in, one out)", timed(lambda: dual_norm_blend(y, w1, gz, w1, 1e-6)),
        nbytes=6 * T * W, like="residual_norm")
    del x
    # --- the convolution in front of every sublayer (4 taps): a row read, a row written
    cu, st0 = i32([0, L]), i32([0])
    slots1, slotsB = i32([1]), i32(list(range(1, B + 1)))
    pre = (N.ptr(cu), N.ptr(st0), None)
    posd = i32([L - 1] * B)
    dec = (None, None, N.ptr(posd))
    hin = torch.randn(L, W, device=dev).to(bf)
    cw = torch.randn(W, TAPS, device=dev) * 0.3
    cstate = torch.zeros(B + 1, TAPS - 1, W, dtype=bf, device=dev)
    cout = torch.empty(L, W, dtype=bf, device=dev)
    add("causal_conv, input + conv (4096 tokens, 4 taps)",
        timed(lambda: N.check(lib.cvllm_causal_conv_mode(N.ptr(hin), W, 0, W, TAPS, N.ptr(cw), None, N.ptr(cstate), *pre,
                                                         N.ptr(slots1), 1, L, N.ptr(cout), W, code, 1, code, st), "conv")),
        nbytes=2 * 2 * L * W, like="causal_conv")
    # --- windowed attention with a distance bias and learned sinks: 32 / 8 heads of 128, window 1024
    H, G, D = 32, 8, HEAD_DIM
    prev = torch.get_default_dtype()
    torch.set_default_dtype(bf)
    try:
        with torch.device(dev):
            attn = BiasedChunkAttention(H, G, D, D, D ** -0.5, sink=True, learned_sink=True, norm=False, window=WINDOW,
                                        bucket_bias=(32, 512))
    finally:
        torch.set_default_dtype(prev)
    with torch.no_grad():
        attn.rel.normal_(0, 0.5)
    attn.refresh_distance_bias()
    cache = PagedKVCache(1, L // PS + 1, (L // PS + 1) * (B + 1) * G, PS, G, D, B + 1, bf, device=dev, v_head_dim=D)
    attn.k_cache, attn.v_cache, attn.page_table, attn.bh_seq_lens = cache.layer_slices(0)
    attn.page_size = PS
    slots = []
    for _ in range(B):
        s = cache.new_batch()
        assert cache.reserve_tokens(s, L + 1) == KVAllocationStatus.SUCCESS
        slots.append(s)
    attn.k_cache.normal_()
    attn.v_cache.normal_()
    set_context(is_prefill=True, cu_seqlens_q=cu, max_seqlen_q=L, max_seqlen_k=L, batch_mapping=i32(slots[:1]),
                positions_i32=torch.arange(L, dtype=torch.int32, device=dev),
                token_slot=torch.full((L,), slots[0], dtype=torch.int32, device=dev), seq_start=st0)
    q = torch.randn(L, H, D, device=dev).to(bf)
    seen = sum(min(i + 1, WINDOW) for i in range(L))        # (query, key) pairs inside the window
    add(f"portion attention, window {WINDOW}, distance bias, sinks (4096 tokens, 32 / 8 heads of 128; mma.sync)",
        timed(lambda: attn.attend(q)), flops=4.0 * D * H * seen, like="bias_attn_varlen_mma (portions, mma.sync)")
    set_context(is_prefill=False, batch_mapping=i32(slots), positions_i32=posd, token_slot=i32(slots), max_seqlen_q=1,
                max_seqlen_k=L)
    qd = torch.randn(B, H, D, device=dev).to(bf)
    add(f"bias_attn_decode, window {WINDOW}, distance bias (8 sequences)", timed(lambda: attn.attend(qd)),
        nbytes=2 * 2 * B * G * WINDOW * D, like="bias_attn_decode")
    reset_context()
    # --- general delta rule: 64 heads of 64 x 64
    Hg, Dg = W // DELTA_DIM, DELTA_DIM
    HD = Hg * Dg
    cols = torch.randn(L, 5 * HD, device=dev).to(bf)
    wraw = torch.randn(L, HD, device=dev).to(bf)
    w0, nw = torch.zeros(HD, device=dev), torch.ones(HD, device=dev)
    gstate = torch.zeros(B + 1, Hg, Dg, Dg, device=dev)
    gout = torch.empty(L, HD, dtype=bf, device=dev)

    def gdelta(geom, bm, Bn, mx_new):
        N.check(lib.cvllm_general_delta(N.ptr(cols), cols.stride(0), 0, HD, 2 * HD, 4 * HD, N.ptr(wraw), HD, N.ptr(w0),
                                        math.exp(-0.5), N.ptr(gstate), 3 * HD, GATE_SIGMOID, N.ptr(nw), Dg, 1e-6, *geom,
                                        N.ptr(bm), Bn, mx_new, N.ptr(gout), HD, Hg, Dg, RESERVED_BATCH, code, st),
                "general_delta")

    add(f"general_delta (one portion of 4096 tokens, {Hg} heads of 64 x 64, with the gated norm)",
        timed(lambda: gdelta(pre, slots1, 1, L)), nbytes=2 * L * HD * 7,
        like="wkv_scan (the same head shape, three key-sized inputs a token against five)")
    rows[-1]["GFLOPs_fp32"] = round(10.0 * Dg * Dg * Hg * L / rows[-1]["ms"] / 1e6, 1)
    add("general_delta (decode, 8 sequences: state read + written)", timed(lambda: gdelta(dec, slotsB, B, 1)),
        nbytes=2 * 4 * B * Hg * Dg * Dg, like="wkv_scan (decode)")
    # --- matrix memory: 32 heads of 128 x 128 (the delta rule's shape in the Fafelix comparison)
    Hm, Dm = W // MEMORY_DIM, MEMORY_DIM
    mcols = torch.randn(L, 4 * Hm * Dm + 2 * Hm, device=dev).to(bf)
    mstate = torch.zeros(B + 1, Hm, Dm, Dm, device=dev)
    nvec, mrun = torch.zeros(B + 1, Hm, Dm, device=dev), torch.zeros(B + 1, Hm, device=dev)
    mnw = torch.ones(Hm * Dm, device=dev)
    mout = torch.empty(L, Hm * Dm, dtype=bf, device=dev)

    def memory(geom, bm, Bn, mx_new):
        i_off = 4 * Hm * Dm
        N.check(lib.cvllm_matrix_memory(N.ptr(mcols), mcols.stride(0), 0, Hm * Dm, 2 * Hm * Dm, i_off, i_off + Hm, 15.0,
                                        Dm ** -0.5, N.ptr(mstate), N.ptr(nvec), N.ptr(mrun), 3 * Hm * Dm, GATE_SIGMOID,
                                        N.ptr(mnw), Dm, 1e-6, *geom, N.ptr(bm), Bn, mx_new, N.ptr(mout), Hm * Dm, Hm, Dm,
                                        Dm, RESERVED_BATCH, code, st), "matrix_memory")

    add(f"matrix_memory (one portion of 4096 tokens, {Hm} heads of 128 x 128, with the gated norm)",
        timed(lambda: memory(pre, slots1, 1, L)), nbytes=2 * L * Hm * Dm * 5,
        like="delta_rule (the same head shape)")
    rows[-1]["GFLOPs_fp32"] = round(4.0 * Dm * Dm * Hm * L / rows[-1]["ms"] / 1e6, 1)
    add("matrix_memory (decode, 8 sequences: state read + written)", timed(lambda: memory(dec, slotsB, B, 1)),
        nbytes=2 * 4 * B * Hm * Dm * Dm, like="delta_rule (decode)")
    # --- selective scan: 8192 channels, 16 state channels each
    inner = 2 * W
    xs = torch.randn(L, inner, device=dev).to(bf)
    dtr = torch.randn(L, inner, device=dev).to(bf)
    zc = torch.randn(L, 2 * inner, device=dev).to(bf)
    dbc = torch.randn(L, DT_RANK + 2 * STATE, device=dev).to(bf)
    dtb, A_log, Dp = torch.full((inner,), -1.0, device=dev), torch.zeros(inner, STATE, device=dev), torch.ones(inner, device=dev)
    sstate = torch.zeros(B + 1, inner, STATE, device=dev)
    sout = torch.empty(L, inner, dtype=bf, device=dev)

    def sscan(geom, bm, Bn, mx_new):
        N.check(lib.cvllm_selective_scan(N.ptr(xs), inner, N.ptr(dtr), inner, N.ptr(dtb), N.ptr(dbc), dbc.stride(0),
                                         DT_RANK, DT_RANK + STATE, N.ptr(A_log), N.ptr(Dp), N.ptr(zc), 2 * inner, inner,
                                         N.ptr(sstate), *geom, N.ptr(bm), Bn, mx_new, N.ptr(sout), inner, inner, STATE,
                                         RESERVED_BATCH, code, st), "selective_scan")

    add(f"selective_scan (one portion of 4096 tokens, {inner} channels x {STATE} states, gate inside)",
        timed(lambda: sscan(pre, slots1, 1, L)), nbytes=2 * L * inner * 4,
        like="ssm_scan + gated_group_norm (the mixer's portion kernel)")
    rows[-1]["G_exp_per_s"] = round(inner * STATE * L / rows[-1]["ms"] / 1e6, 1)
    add("selective_scan (decode, 8 sequences: state read + written)", timed(lambda: sscan(dec, slotsB, B, 1)),
        nbytes=2 * 4 * B * inner * STATE, like="ssm_scan (decode)")
    return rows


def run(peaks: dict, sizes: List[str], reps: int) -> dict:
    from compactor_vllm.config.model_config import BatasunConfig, FafelixConfig, NununexConfig

    result = {"arch": "nununex", "closest": "fafelix (pair embedding, attention with learned sinks, matrix-state "
                                            "mixers); batasun for the state-space layers and the routed experts",
              "dtype": "bf16", "data": "synthetic (random weights)",
              "workload": {"prefill_tokens": PREFILL_TOKENS, "decode_batch": DECODE_BATCH,
                           "decode_context": DECODE_CONTEXT, "decode_steps": DECODE_STEPS}, "sizes": {}}
    for name in sizes:
        s = SIZES[name]
        row = {"shape": s}
        row["fafelix_attention_only"] = engine_throughput("fafelix", FafelixConfig.from_json(fafelix_config(s, "A")), reps)
        row["fafelix_wkv_only"] = engine_throughput("fafelix", FafelixConfig.from_json(fafelix_config(s, "W")), reps)
        row["fafelix_mixed"] = engine_throughput("fafelix", FafelixConfig.from_json(fafelix_config(s, "AWDA")), reps)
        row["batasun_state_space_only"] = engine_throughput("batasun", BatasunConfig.from_json(batasun_config(s, "M")), reps)
        for label, pattern, moe in (("nununex_parallel_only", "P", False), ("nununex_general_delta_only", "G", False),
                                    ("nununex_selective_scan_only", "S", False), ("nununex_mixed", "SGPG", False),
                                    ("nununex_selective_scan_only_moe", "S", True)):
            row[label] = engine_throughput("nununex", NununexConfig.from_json(nununex_config(s, pattern, moe)), reps)
        result["sizes"][name] = row
    result["kernels"] = kernel_rooflines(peaks, max(reps, 5))
    result["peaks"] = peaks
    return result


def main(peaks: dict, sizes: str, reps: int) -> None:
    print(json.dumps(run(peaks, [x for x in sizes.split(",") if x], reps)))
