"""Prefill and decode throughput of a Movolorn model beside a Qwen3 model of equal size (random weights), both through
the engine's runner, plus the new kernels timed alone against the measured peaks.

Used by `bench.py --arch movolorn`; the default workload of bench.py does not touch this module.
Timing: CUDA events on the launching stream, after warm-up; between timed kernel iterations a buffer larger than L2 is
written.  Engine-level numbers include the runner's host work (scheduling, index vectors), as a user sees them.
"""
from __future__ import annotations

import json
import math
from types import SimpleNamespace
from typing import Callable, Dict, List

import torch

SIZES = {
    # name: width, heads, kv heads, ff, layers, vocab
    "1b-like": dict(width=2048, heads=16, kv_heads=4, ff=8192, layers=4, vocab=32000),
    "8b-like": dict(width=4096, heads=32, kv_heads=8, ff=14336, layers=2, vocab=32000),
}
HEAD_DIM = 128           # the size the 16-bit prefill / decode kernels of the other models serve
PREFILL_TOKENS = 4096
DECODE_BATCH, DECODE_CONTEXT, DECODE_STEPS = 8, 2048, 64


def movolorn_config(s: dict, chunk: int, moe: bool) -> dict:
    mixer = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": HEAD_DIM, "vdim": HEAD_DIM,
             "scale": HEAD_DIM ** -0.5}
    if chunk:
        mixer["mask"] = {"size": chunk}
    if moe:   # 8 experts of a quarter of the dense size, 2 per token, plus a shared one: about the dense layer's work
        mlp = {"kind": "moe", "expert": {"ff": s["ff"] // 4}, "shared": {"ff": s["ff"] // 2},
               "router": {"experts": 8, "identity": 0, "top": 2, "groups": {"count": 2, "keep": 1}}}
    else:
        mlp = {"kind": "dense", "ff": s["ff"]}
    return {"architecture": "Movolorn", "vocab": s["vocab"], "width": s["width"], "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": [{"type": "attention", "mixer": mixer, "mlp": mlp}] * s["layers"]}


def qwen3_config(s: dict):
    return SimpleNamespace(
        model_type="qwen3", vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"],
        num_hidden_layers=s["layers"], num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"],
        head_dim=HEAD_DIM, rms_norm_eps=1e-6, rope_theta=1e6, rope_scaling=None, max_position_embeddings=1 << 16,
        torch_dtype=torch.bfloat16, tie_word_embeddings=False, attention_bias=False)


def _events_ms(fn: Callable[[], None], reps: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sorted(times)[len(times) // 2]


def engine_throughput(kind: str, hf, reps: int) -> Dict[str, float]:
    """tokens/s of one PREFILL_TOKENS prompt, and of DECODE_BATCH sequences decoding at DECODE_CONTEXT."""
    from compactor_vllm.api_types import (BatchCompressionParams, CompressionMethod, SamplingParams,
                                          SequenceCompressionParams)
    from compactor_vllm.config.engine_config import LLMConfig
    from compactor_vllm.core.model_runner import ModelRunner
    from compactor_vllm.utils.sequence import Sequence

    page = 128
    need = PREFILL_TOKENS + DECODE_BATCH * (DECODE_CONTEXT + DECODE_STEPS + page)
    heads = hf.num_key_value_heads
    cfg = LLMConfig(model="synthetic", hf_config=hf, dtype=None if kind == "qwen3" else "bfloat16",
                    max_num_seqs=DECODE_BATCH, max_model_len=8192, kvcache_page_size=page, eos=-1)
    pages = need // page + 8
    runner = ModelRunner(cfg, num_pages=pages * heads if kind == "qwen3" else pages, seed=1,
                         max_batched_tokens=8192)
    none = BatchCompressionParams(compression_method=CompressionMethod.NONE, do_chunked_compression=False)
    g = torch.Generator().manual_seed(0)
    vocab = hf.vocab_size

    def seq(n, new):
        return Sequence(prompt_token_ids=torch.randint(0, vocab, (n,), generator=g).tolist(),
                        sampling_params=SamplingParams(temperature=0.0, max_new_tokens=new),
                        compression_params=SequenceCompressionParams(1.0))

    def prefill():
        runner.generate([seq(PREFILL_TOKENS, 1)], none)

    def decode(new):
        runner.generate([seq(DECODE_CONTEXT, new) for _ in range(DECODE_BATCH)], none)

    out = {"prefill_ms": _events_ms(prefill, reps)}
    out["prefill_tok_s"] = PREFILL_TOKENS / out["prefill_ms"] * 1e3
    short = _events_ms(lambda: decode(1), max(2, reps // 2), warmup=2)
    long = _events_ms(lambda: decode(1 + DECODE_STEPS), max(2, reps // 2), warmup=2)
    out["decode_ms_per_step"] = (long - short) / DECODE_STEPS
    out["decode_tok_s"] = DECODE_BATCH / out["decode_ms_per_step"] * 1e3
    out["graph_replays"] = runner.stats["graph_replays"]
    del runner
    torch.cuda.empty_cache()
    return out


def kernel_rooflines(peaks: dict, reps: int) -> List[dict]:
    """The new kernels alone at HQ = 32, HKV = 8, D = 128, width 4096, bfloat16: achieved rate and its fraction of
    the measured copy bandwidth / cuBLAS bf16 rate."""
    from compactor_vllm import _native as N
    from compactor_vllm.kv_cache.page_table import PagedKVCache
    from compactor_vllm.layers.attention import BiasedChunkAttention, linear_bias_slopes
    from compactor_vllm.layers.layernorm import sandwich_norm
    from compactor_vllm.layers.moe import ACT_SILU, gated_act, route
    from compactor_vllm.utils.context import reset_context, set_context

    dev = torch.device("cuda", torch.cuda.current_device())
    bf = torch.bfloat16
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    hbm = float(peaks["hbm"]) * 1e9                 # GB/s of the copy measurement (bench.py peaks())
    tflops = float(peaks["tensor_burst"]) * 1e12    # cuBLAS bf16 burst: the kernels are timed alone
    rows: List[dict] = []

    def timed(fn):
        def run():
            flush_buf.zero_()
            fn()
        with_flush = _events_ms(run, reps)
        only_flush = _events_ms(lambda: flush_buf.zero_(), reps)
        return max(with_flush - only_flush, 1e-4)

    def add(name, ms, *, nbytes=None, flops=None, like=None):
        r = {"kernel": name, "ms": round(ms, 4), "like": like}
        if nbytes is not None:
            r["GBs"] = round(nbytes / ms / 1e6, 1)
            r["frac_hbm_of_measured"] = round(nbytes / (ms * 1e-3) / hbm, 3)
        if flops is not None:
            r["TFLOPs"] = round(flops / ms / 1e9, 1)
            r["frac_bf16_of_measured"] = round(flops / (ms * 1e-3) / tflops, 4)
        rows.append(r)

    T, W, H, G, D, PS = 8192, 4096, 32, 8, 128, 128
    # sandwich norm: branch (2 B) + residual read and write (8 B) + normed output (2 B) per element
    x = torch.randn(T, W, device=dev)
    y = torch.randn(T, W, device=dev).to(bf)
    w1, w2 = torch.ones(W, device=dev), torch.ones(W, device=dev)
    add("sandwich_norm", timed(lambda: sandwich_norm(x, branch=y, post_weight=w1, pre_weight=w2, out_dtype=bf)),
        nbytes=12 * T * W, like="rmsnorm_kernel (fused add + norm)")
    del x, y
    # gated activation: 2 x F in, F out, 16 bit
    F_ = 14336
    gu = torch.randn(T, 2 * F_, device=dev).to(bf)
    add("gated_act", timed(lambda: gated_act(gu, ACT_SILU)), nbytes=6 * T * F_, like="torch silu * up (2 launches)")
    del gu
    # router: fp32 logits in, indices and weights out
    E = 64
    lg = torch.randn(T * 4, E, device=dev)
    add("moe_route", timed(lambda: route(lg, None, 6, 8, 4)), nbytes=4 * T * 4 * (E + 12), like=None)
    # attention over the paged cache
    L = 4096
    attn = BiasedChunkAttention(H, G, D, D, D ** -0.5, slopes=linear_bias_slopes(H), chunk=0, sink=True, qk_norm=True)
    attn = attn.to(dev)
    cache = PagedKVCache(1, L // PS + 1, G * (L // PS + 1) * 9, PS, G, D, 9, bf, device=dev)
    attn.k_cache, attn.v_cache, attn.page_table, attn.bh_seq_lens = cache.layer_slices(0)
    attn.page_size = PS
    from compactor_vllm.kv_cache.page_table import KVAllocationStatus
    slots = []
    for _ in range(8):
        s = cache.new_batch()
        assert cache.reserve_tokens(s, L + 1) == KVAllocationStatus.SUCCESS
        slots.append(s)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    qkv = torch.randn(L, (H + 2 * G) * D, device=dev).to(bf)

    def prefill_ctx(chunk):
        attn.chunk = chunk
        set_context(is_prefill=True, cu_seqlens_q=i32([0, L]), max_seqlen_q=L, batch_mapping=i32(slots[:1]),
                    positions_i32=torch.arange(L, dtype=torch.int32, device=dev),
                    token_slot=torch.full((L,), slots[0], dtype=torch.int32, device=dev), seq_start=i32([0]))

    lib, code = N.lib(), N.CVLLM_BF16
    q = torch.empty(L, H, D, dtype=bf, device=dev)
    out = torch.empty(L, H, D, dtype=bf, device=dev)
    pt = attn.page_table
    table = (N.ptr(pt), pt.stride(0), pt.stride(1), PS)
    from compactor_vllm.utils.context import get_context

    def store():
        c = get_context()
        N.check(lib.cvllm_qknorm_store(N.ptr(qkv), qkv.stride(0), N.ptr(attn.q_norm_weight), N.ptr(attn.k_norm_weight),
                                       1e-6, N.ptr(c.positions_i32), N.ptr(c.token_slot), N.ptr(q), N.ptr(attn.k_cache),
                                       N.ptr(attn.v_cache), *table, N.ptr(attn.bh_seq_lens), L, H, G, D, D, 0, code,
                                       N.stream(dev)), "store")

    def varlen():
        c = get_context()
        N.check(lib.cvllm_bias_attn_varlen(N.ptr(q), N.ptr(attn.k_cache), N.ptr(attn.v_cache), *table,
                                           N.ptr(c.cu_seqlens_q), N.ptr(c.seq_start), N.ptr(c.batch_mapping),
                                           N.ptr(attn.slopes), attn.chunk, 1, None, attn.scale, N.ptr(out), 1, L, H, G,
                                           D, D,
                                           L, attn.k_cache.shape[0], pt.shape[-1], 0, code, N.stream(dev)), "varlen")

    prefill_ctx(0)
    add("qknorm_store", timed(store), nbytes=2 * L * ((H + 2 * G) * D + (H + 2 * G) * D),
        like="rope_qk_kernel with q/k norm + store_all_kernel")
    add("bias_attn_varlen (no chunk, 4096 tokens)", timed(varlen), flops=4.0 * D * H * L * (L + 1) / 2,
        like="prefill_attn2_kernel")
    prefill_ctx(1024)
    add("bias_attn_varlen (chunk 1024, 4096 tokens)", timed(varlen), flops=4.0 * D * H * (L // 1024) * 1024 * 1025 / 2,
        like="prefill_attn2_kernel")
    # decode: 8 sequences at position L - 1 (every slot's cache row range is allocated; the contents do not matter)
    B = 8
    qd = torch.randn(B, H, D, device=dev).to(bf)
    od = torch.empty(B, H, D, dtype=bf, device=dev)
    pos, bm = i32([L - 1] * B), i32(slots)

    def decode(chunk):
        attn.chunk = chunk
        splits = attn.decode_splits(B, L)
        ws = N.workspace(dev, 4 * B * H * splits * (2 + D), "bias_attn_decode")
        N.check(lib.cvllm_bias_attn_decode(N.ptr(qd), N.ptr(attn.k_cache), N.ptr(attn.v_cache), *table, N.ptr(pos),
                                           N.ptr(bm), N.ptr(attn.slopes), chunk, 1, None, attn.scale, N.ptr(od), B, H, G,
                                           D, D,
                                           0, splits, N.ptr(ws), ws.numel(), 0, code, N.stream(dev)), "decode")

    add("bias_attn_decode (no chunk, 8 x 4096)", timed(lambda: decode(0)), nbytes=2 * 2 * B * G * L * D,
        like="decode_attn_kernel")
    add("bias_attn_decode (chunk 1024, 8 x 1024)", timed(lambda: decode(1024)), nbytes=2 * 2 * B * G * 1024 * D,
        like="decode_attn_kernel")
    reset_context()
    # expert products for a decode step: 8 tokens x 2 choices, experts of ff 3584 at width 4096
    Fe, Ee, top = 3584, 8, 2
    wgu = torch.randn(Ee, 2 * Fe, W, device=dev).to(bf)
    xs = torch.randn(B, W, device=dev).to(bf)
    idx = torch.randint(0, Ee, (B * top,), device=dev, dtype=torch.int32)
    a = torch.empty(B * top, Fe, dtype=bf, device=dev)
    add("expert_gemv (gate | up, 16 pairs)",
        timed(lambda: N.check(lib.cvllm_expert_gemv(N.ptr(xs), top, N.ptr(wgu), N.ptr(idx), Ee, N.ptr(a), B * top, Fe, W,
                                                    0, 0.0, code, N.stream(dev)), "gemv")),
        nbytes=2 * B * top * 2 * Fe * W, like="cuBLAS GEMV-shaped GEMM of the dense models")
    return rows


def run(peaks: dict, sizes: List[str], reps: int) -> dict:
    from compactor_vllm.config.model_config import MovolornConfig

    result = {"arch": "movolorn", "closest": "qwen3", "dtype": "bf16", "data": "synthetic (random weights)",
              "workload": {"prefill_tokens": PREFILL_TOKENS, "decode_batch": DECODE_BATCH,
                           "decode_context": DECODE_CONTEXT, "decode_steps": DECODE_STEPS}, "sizes": {}}
    for name in sizes:
        s = SIZES[name]
        row = {"shape": s}
        row["qwen3"] = engine_throughput("qwen3", qwen3_config(s), reps)
        for label, chunk, moe in (("movolorn_dense_nochunk", 0, False), ("movolorn_dense_chunk1024", 1024, False),
                                  ("movolorn_moe_chunk1024", 1024, True)):
            row[label] = engine_throughput("movolorn", MovolornConfig.from_json(movolorn_config(s, chunk, moe)), reps)
        result["sizes"][name] = row
    result["kernels"] = kernel_rooflines(peaks, max(reps, 5))
    result["peaks"] = peaks
    return result


def main(peaks: dict, sizes: str, reps: int) -> None:
    print(json.dumps(run(peaks, [x for x in sizes.split(",") if x], reps)))
