"""Attention module — the drop-in boundary (reference: layers/attention.py:17-161).

Prefill: store of the new K/V (all rows, or only the top-scoring (token, head)
pairs) on STORE_STREAM concurrently with causal attention over
[cached prefix || new K/V] on the main stream.  Decode: append one row per
(b, h), then split-KV paged attention.  The KV-cache manager injects k_cache,
v_cache, page_table, bh_seq_lens and page_size (core/memory_manager.py).
"""
from typing import Optional

import torch
from compactor_vllm.attention.sparse_decode_kernel import decode_append_and_attend, head_sparse_decode_attention
from compactor_vllm.attention.sparse_varlen_kernel import causal_sparse_varlen_with_cache
from compactor_vllm.compression.common import extract_and_store_top_kv
from compactor_vllm.config.constants import RESERVED_BATCH
from compactor_vllm.config.engine_config import AttentionBackend
from compactor_vllm.kv_cache.store_kv_cache import decode_store_kv, prefill_store_all_kv
from compactor_vllm.utils.context import Context, get_context
from compactor_vllm.utils.helpers import maybe_execute_in_stream
from torch import nn


class Attention(nn.Module):
    def __init__(self, num_heads, head_dim, scale, num_kv_heads):
        super().__init__()
        self.num_heads: int = num_heads
        self.head_dim = head_dim
        self.scale: float = scale
        self.num_kv_heads = int(num_kv_heads)
        self.k_cache: Optional[torch.Tensor] = None
        self.v_cache: Optional[torch.Tensor] = None
        self.page_table: Optional[torch.Tensor] = None
        self.bh_seq_lens: Optional[torch.Tensor] = None
        self.page_size: Optional[int] = None

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scores: Optional[torch.Tensor] = None):
        context: Context = get_context()
        batch_mapping = context.batch_mapping
        if not context.is_prefill and self.bh_seq_lens is not None and self.bh_seq_lens.is_contiguous():
            # decode: append + attend index bh_seq_lens through batch_mapping themselves — the
            # reference's index_select / index_copy_ round trip (:46-50,152-160) is not needed
            assert self.k_cache is not None, "KV Cache must be initialized for decoding"
            return decode_append_and_attend(
                q, k, v, self.k_cache, self.v_cache, self.bh_seq_lens, self.page_table, batch_mapping,
                int(self.num_kv_heads), self.page_size, self.scale, reserved_batch=RESERVED_BATCH,
            )
        seq_lens = (
            None if self.bh_seq_lens is None
            else self.bh_seq_lens.index_select(0, batch_mapping).contiguous()
        )
        if context.is_prefill:
            # attention must see the PRE-store lengths (reference :52,115)
            seq_lens_copy = seq_lens.clone() if seq_lens is not None else None
            if self.k_cache is not None and context.do_compression and scores is not None:
                cc = context.compression_context
                assert cc is not None
                maybe_execute_in_stream(
                    extract_and_store_top_kv,
                    scores=scores, cu_seqlens_k=context.cu_seqlens_k, max_k_len=context.max_seqlen_k,
                    top_k=cc.max_tokens_to_retain, H=int(self.num_kv_heads), new_keys=k, new_vals=v,
                    num_tokens_to_retain=cc.batch_tokens_to_retain, page_table=self.page_table,
                    batch_mapping=batch_mapping, bh_lens=seq_lens, k_cache=self.k_cache,
                    v_cache=self.v_cache, PAGE_SIZE=self.page_size, PAD_TO_PAGE_SIZE=True,
                    STORE_STREAM=context.STORE_STREAM,
                )
            elif self.k_cache is not None:
                maybe_execute_in_stream(
                    prefill_store_all_kv,
                    new_keys=k, new_values=v, cu_seqlens_k=context.cu_seqlens_k,
                    max_seqlen_k=context.max_seqlen_k, k_cache=self.k_cache, v_cache=self.v_cache,
                    page_table=self.page_table, bh_lens=seq_lens, batch_mapping=batch_mapping,
                    PAGE_SIZE=self.page_size, STORE_STREAM=context.STORE_STREAM,
                )
            if context.attention_backend == AttentionBackend.FLASH_ATTENTION:
                # The reference dispatches to flash-attn here (:96-107).  This build has one
                # backend by design (no multi-backend dispatch); fail loudly rather than fall back.
                raise NotImplementedError(
                    "AttentionBackend.FLASH_ATTENTION is not provided; use COMPACTOR_TRITON "
                    "(served by the sm_100a CUDA kernels)"
                )
            elif context.attention_backend == AttentionBackend.COMPACTOR_TRITON:
                o = causal_sparse_varlen_with_cache(
                    q, k, v, self.k_cache, self.v_cache,
                    seq_lens_bh=seq_lens_copy, global_page_table=self.page_table,
                    batch_mapping=batch_mapping, cu_seqlens_q=context.cu_seqlens_q,
                    max_seqlen_q=context.max_seqlen_q, max_seqlen_k_cache=context.max_bh_len,
                    HKV=int(self.num_kv_heads), PAGE_SIZE=self.page_size, sm_scale=self.scale,
                )
            else:
                raise NotImplementedError
        else:
            assert self.k_cache is not None, "KV Cache must be initialized for decoding"
            decode_store_kv(
                key=k, value=v, batch_mapping=batch_mapping, bh_lens=seq_lens,
                page_table=self.page_table, k_cache=self.k_cache, v_cache=self.v_cache,
                PAGE_SIZE=self.page_size,
            )
            o = head_sparse_decode_attention(
                q, self.k_cache, self.v_cache, seq_lens, self.page_table, batch_mapping,
                int(self.num_kv_heads), self.page_size, self.scale, key_split=context.key_split,
            )
        if self.bh_seq_lens is not None:
            maybe_execute_in_stream(
                self.bh_seq_lens.index_copy_, 0, batch_mapping.to(torch.long), seq_lens,
                STORE_STREAM=context.STORE_STREAM if context.is_prefill else None,
            )
        return o


def linear_bias_slopes(num_heads: int, base_exponent: float = 8.0) -> torch.Tensor:
    """Per-head slopes of a linear distance bias: slope_h = 2 ** (-base_exponent * (h + 1) / num_heads), fp32."""
    h = torch.arange(1, num_heads + 1, dtype=torch.float64)
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), -base_exponent * h / num_heads).float()


def pair_rotation_frequencies(dims: int, base: float, scaling: Optional[tuple] = None) -> torch.Tensor:
    """Rotation frequencies of dims / 2 pairs as 64-bit floats: f_i = base ** (-2 i / dims).  `scaling` =
    (factor, low, high, original) stretches long wavelengths: with l = 2 pi / f, f stays where l < original / high,
    becomes f / factor where l > original / low, and between the two is blended with
    s = (original / l - low) / (high - low):  (1 - s) f / factor + s f."""
    import math

    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = (float(v) for v in scaling)
            wavelength = 2.0 * math.pi / f
            if wavelength > original / low:
                f = f / factor
            elif wavelength >= original / high:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def distance_buckets(rows: int, far: int, length: int) -> list:
    """Row of a learned distance-bias table of `rows` rows for the distances 0 .. length - 1: distances below
    rows // 2 have a row each, larger ones share logarithmic buckets that reach the last row at distance `far`:
    bucket(n) = min(rows - 1, half + floor(ln(n / half) / ln(far / half) * (rows - half))), half = rows // 2."""
    import math

    half = rows // 2
    out = []
    for n in range(length):
        if n < half or half == 0:
            out.append(min(n, rows - 1))
        elif far <= half:           # no room for logarithmic buckets: everything from `half` on shares the last row
            out.append(rows - 1)
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


class BiasedChunkAttention(nn.Module):
    """Attention over the paged cache for models without rotation (csrc/bias_attn.cu):

        score(i, j) = scale * q_i . k_j - slopes[h] * (i - j),   j <= i and floor(i / chunk) == floor(j / chunk)
        p_j = exp(score_j) / (sink * exp(sink_logits[h]) + sum_j exp(score_j))

    with optional per-head RMS norm of q and k (weights shared by all heads, or none), any head sizes (value size may
    differ from the key size) and bfloat16 or float32 storage.  `slopes` None = no bias, `chunk` 0 = plain causal,
    `sink` False = plain softmax; `learned_sink` gives every head its own sink score (a parameter, not scaled; without
    it the score is 0).  `rotation` (inv_freq [rot_dims / 2] float64, see `pair_rotation_frequencies`) turns
    neighbouring pairs (2 i, 2 i + 1) of the first rot_dims numbers of every q and k head by position * inv_freq[i]
    BEFORE the norm; `norm` False leaves q and k unnormed.  `window` > 0: a query sees only the keys at distances
    0 .. window - 1.  `bucket_bias` = (rows, far): a learned table `rel` [rows, H] adds rel[bucket(i - j), h] to the
    score (unscaled; buckets as in `distance_buckets`); the kernels read it spread out per distance (`dist_bias`,
    rebuilt by `refresh_distance_bias()` whenever `rel` changes).  forward() takes the packed projection rows
    [T, H*D + G*D + G*Dv] (row stride free): one launch rotates / norms q / k
    and writes k / v to the cache at the tokens' positions, one launch attends — the portion kernel when any
    sequence of the step brings more than one token, the decode kernel otherwise.  The step's geometry comes from the
    global context: `positions_i32`, `token_slot`, `cu_seqlens_q`, `seq_start`, `batch_mapping`, `max_seqlen_q`.
    The cache manager injects the cache views exactly as for `Attention`."""

    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, scale: float, *,
                 slopes: Optional[torch.Tensor] = None, chunk: int = 0, sink: bool = False, qk_norm: bool = False,
                 eps: float = 1e-6, values_in_keys: bool = False, learned_sink: bool = False,
                 rotation: Optional[torch.Tensor] = None, norm: bool = True, window: int = 0,
                 bucket_bias: Optional[tuple] = None):
        super().__init__()
        self.norm = bool(norm)
        self.window = int(window)
        self.bias_far = 0
        self.rel = None
        if bucket_bias is not None:
            rows, self.bias_far = int(bucket_bias[0]), int(bucket_bias[1])
            self.rel = nn.Parameter(torch.zeros(rows, num_heads, dtype=torch.float32))
        self.register_buffer("dist_bias", None, persistent=False)
        self.sink_logits = nn.Parameter(torch.zeros(num_heads, dtype=torch.float32)) if learned_sink else None
        if rotation is not None:
            assert rotation.dtype == torch.float64 and 2 * rotation.numel() <= head_dim
        self.register_buffer("inv_freq", None if rotation is None else rotation.contiguous(), persistent=False)
        # values_in_keys: a value row is the first v_head_dim columns of its key row; there is no value cache
        self.values_in_keys = bool(values_in_keys)
        self.num_heads, self.num_kv_heads = int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale, self.chunk, self.sink, self.eps = float(scale), int(chunk), bool(sink), float(eps)
        self.register_buffer("slopes", None if slopes is None else slopes.float().contiguous(), persistent=False)
        self.q_norm_weight = nn.Parameter(torch.ones(head_dim, dtype=torch.float32)) if qk_norm else None
        self.k_norm_weight = nn.Parameter(torch.ones(head_dim, dtype=torch.float32)) if qk_norm else None
        self.k_cache: Optional[torch.Tensor] = None
        self.v_cache: Optional[torch.Tensor] = None
        self.page_table: Optional[torch.Tensor] = None
        self.bh_seq_lens: Optional[torch.Tensor] = None
        self.page_size: Optional[int] = None

    @torch.no_grad()
    def refresh_distance_bias(self, rel: Optional[torch.Tensor] = None) -> None:
        """`rel` (given: the new table, any number of rows) spread out per distance: dist_bias[n, h] =
        rel[bucket(n), h] for n up to where the buckets (or the window) end; larger distances read the last row."""
        if rel is not None:
            self.rel = nn.Parameter(rel.detach().to(device=self.rel.device, dtype=torch.float32).contiguous())
        rows = self.rel.shape[0]
        length = max(self.bias_far, rows // 2) + 1
        if self.window > 0:
            length = min(length, self.window)
        idx = torch.tensor(distance_buckets(rows, self.bias_far, max(length, 1)), dtype=torch.long, device=self.rel.device)
        self.dist_bias = self.rel.detach().index_select(0, idx).contiguous()

    @property
    def qkv_width(self) -> int:
        return (self.num_heads + self.num_kv_heads) * self.head_dim + self.num_kv_heads * self.v_head_dim

    def decode_splits(self, batch: int, max_keys: int) -> int:
        """Parts a sequence's keys are cut into for a decode step.  Small steps: as many as fill ONE wave of two CTAs
        per SM (148 SMs) with at least 128 keys per part.  Large steps (many sequences or long contexts) run faster
        with several waves of shorter CTAs while a part keeps 1024 keys: measured at 32 / 8 heads of 128, 8 x 16384
        keys 1.75 -> 2.05 TB/s (4 -> 16 parts), 32 x 4096 keys 1.74 -> 2.15 TB/s (1 -> 4 parts); thinner parts lose
        again to the merge pass when the bound `max_keys` is well above the keys really there (graph replays).
        `max_keys` bounds the keys a query can see (the chunk bounds it further)."""
        keys = min(max_keys, self.chunk) if self.chunk else max_keys
        if self.window:
            keys = min(keys, self.window)
        ctas = max(batch * self.num_kv_heads * -(-(self.num_heads // self.num_kv_heads) // 4), 1)
        one_wave = min(296 // ctas, keys // 128)
        several = min(2048 // ctas, keys // 1024)
        return int(max(1, min(max(one_wave, several), 64)))

    def forward(self, qkv: torch.Tensor) -> torch.Tensor:
        from compactor_vllm import _native as N

        ctx: Context = get_context()
        assert self.k_cache is not None, "KV cache must be initialized"
        T = qkv.shape[0]
        H, G, D, Dv = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        assert qkv.shape[1] == self.qkv_width and qkv.stride(1) == 1 and qkv.dtype == self.k_cache.dtype
        dev, code, lib = qkv.device, N.block_dtype_code(qkv.dtype), N.lib()
        q = torch.empty((T, H, D), dtype=qkv.dtype, device=dev)
        pt = self.page_table
        table = (N.ptr(pt), pt.stride(0), pt.stride(1), int(self.page_size))
        rot = self.inv_freq
        N.check(lib.cvllm_rope_qknorm_store(
            N.ptr(qkv), qkv.stride(0), N.ptr(rot), 0 if rot is None else 2 * rot.numel(), int(self.norm),
            N.ptr(self.q_norm_weight), N.ptr(self.k_norm_weight), self.eps,
            N.ptr(ctx.positions_i32), N.ptr(ctx.token_slot), N.ptr(q), N.ptr(self.k_cache), N.ptr(self.v_cache),
            *table, N.ptr(self.bh_seq_lens), T, H, G, D, Dv, RESERVED_BATCH, code, N.stream(dev)),
            "cvllm_rope_qknorm_store")
        return self.attend(q)

    def attend(self, q: torch.Tensor, flat: bool = True) -> torch.Tensor:
        """q [T, H, D] (normed / rotated already, the step's keys in the cache) -> [T, H * Dv], or with flat=False
        [T, H, Dv] (possibly a view of wider rows)."""
        from compactor_vllm import _native as N

        ctx: Context = get_context()
        T = q.shape[0]
        H, G, D, Dv = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        assert q.is_contiguous() and q.dtype == self.k_cache.dtype
        dev, code, lib = q.device, N.block_dtype_code(q.dtype), N.lib()
        pt = self.page_table
        table = (N.ptr(pt), pt.stride(0), pt.stride(1), int(self.page_size))
        v_cache, v_stride = (self.k_cache, D) if self.values_in_keys else (self.v_cache, Dv)
        keep = Dv
        if (self.values_in_keys and ctx.is_prefill and q.dtype == torch.bfloat16 and D == 128 and Dv < D
                and self.page_size % 128 == 0 and (H // G) % 2 == 0):
            # Values that are columns of 128-wide key rows: taking the WHOLE row as the value costs a few more
            # products and puts the portion on the tcgen05 pipeline (which serves D = Dv = 128); the columns past
            # the values are dropped on return.
            Dv = D
        out = torch.empty((T, H, Dv), dtype=q.dtype, device=dev)
        if self.rel is not None and self.dist_bias is None:
            self.refresh_distance_bias()
        db = self.dist_bias
        dist = (self.window, N.ptr(db), 0 if db is None else db.shape[0])
        if ctx.is_prefill:
            B = ctx.batch_mapping.numel()
            N.check(lib.cvllm_bias_attn_varlen_dist(
                N.ptr(q), N.ptr(self.k_cache), N.ptr(v_cache), *table, N.ptr(ctx.cu_seqlens_q),
                N.ptr(ctx.seq_start), N.ptr(ctx.batch_mapping), N.ptr(self.slopes), self.chunk, *dist, int(self.sink),
                N.ptr(self.sink_logits), self.scale, N.ptr(out), B, int(ctx.max_seqlen_q), H, G, D, Dv, T, self.k_cache.shape[0], pt.shape[-1],
                v_stride, code, N.stream(dev)), "cvllm_bias_attn_varlen")
        else:
            assert ctx.batch_mapping.numel() == T
            splits = self.decode_splits(T, int(ctx.max_seqlen_k))
            ws = N.workspace(dev, 4 * T * H * splits * (2 + Dv), "bias_attn_decode") if splits > 1 else None
            N.check(lib.cvllm_bias_attn_decode_dist(
                N.ptr(q), N.ptr(self.k_cache), N.ptr(v_cache), *table, N.ptr(ctx.positions_i32),
                N.ptr(ctx.batch_mapping), N.ptr(self.slopes), self.chunk, *dist, int(self.sink), N.ptr(self.sink_logits),
                self.scale, N.ptr(out), T, H, G, D, Dv, RESERVED_BATCH, splits, N.ptr(ws), ws.numel() if ws is not None else 0, v_stride, code,
                N.stream(dev)), "cvllm_bias_attn_decode")
        if keep != Dv:
            out = out[:, :, :keep]
            return out.reshape(T, H * keep) if flat else out
        return out.view(T, H * Dv) if flat else out
