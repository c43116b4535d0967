"""Mixers whose state is one [key, value] matrix per head, carried from token to token (csrc/recurrent.cu).

`DeltaRuleMixer`, the gated delta rule.  From the columns [q | k | v | gate | beta | decay] of a projection of the
layer's input: q, k (kv_heads x dim) and v (heads x vdim) pass a short causal convolution per channel and silu; q and k
become unit vectors per head (q times dim^-1/2); per head, with beta = sigmoid(.) and g = exp(-exp(A_log) *
softplus(. + dt_bias)):
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
then each head's o is divided by its root mean square, multiplied by a weight (one vector for all heads) and by
silu(gate), and goes through W_o.

`WkvMixer`, time mixing with a per-channel decay.  With h' the previous token's input, each of r, k, v, gate, w reads
its own blend h + (h' - h) mu; r, k, v, gate are projections of their blends (heads x dim), the decay is
w = exp(-exp(W_2 tanh(W_1 blend_w) + w0)); per head
    o = (S + diag(bonus) k v^T)^T r;   S <- diag(w) S + k v^T
then the same unit norm per head, a weight (one per channel), silu(gate) and W_o.

`GeneralDeltaMixer`, a delta rule with a decay and a removal rate per key channel.  From the columns
[r | k | v | gate | a | w1] of a projection of its input: w = exp(-rate * sigmoid(W_2 tanh(w1) + w0)), a = sigmoid(a),
u = k / sqrt(sum k^2 + 1e-6) per head;
    S <- diag(w) S - (a u)(u^T S) + k v^T  (both terms read the old S);   o = S^T r
then the unit norm per head, a weight per channel, sigmoid(gate) and W_o.

`MatrixMemoryMixer`, a matrix memory with exponential gates.  From the columns [q | k | v | gate | i | f] (i, f one
logit per head, biased): i = cap tanh(i / cap), f = logsigmoid(cap tanh(f / cap)), and with a running maximum m that
starts at 0
    m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;  n <- the same with k alone;
    o = S^T q / (max(|n . q|, exp(-m')) + 1e-6),   q times dim^-1/2
then the same unit norm, weight, sigmoid(gate).  Its W_o belongs to the caller's arrangement (`o_proj`).

The recurrence, decays, gates of the recurrence, unit norms and the state are fp32; projections and convolution inputs
are in the model's type.  What a sequence carries between steps (the matrix state, the convolution's last inputs, the
previous token's input) lives in a `MixerState`, whose tensors the state pool allocates per slot; a layer that runs
several times per token owns one `MixerState` per run.  A portion that starts at position 0 starts from zeros.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
from torch import nn

from compactor_vllm import _native as N
from compactor_vllm.config.constants import RESERVED_BATCH
from compactor_vllm.utils.context import get_context


class MixerState(nn.Module):
    """Holder of one run's state tensors ([slots, *shape] each, set as attributes by the state pool)."""

    def __init__(self, specs: Dict[str, Tuple[tuple, Optional[torch.dtype]]]):
        super().__init__()
        self._specs = dict(specs)
        for name in specs:
            setattr(self, name, None)

    def state_specs(self, dtype: torch.dtype):
        return {k: (shape, dtype if dt is None else dt) for k, (shape, dt) in self._specs.items()}


def _geometry(ctx):
    """(cu_seqlens_q, seq_start, positions) pointers of the step, B, the longest portion."""
    portions = ctx.is_prefill      # else: one token per sequence, at positions_i32
    geom = ((N.ptr(ctx.cu_seqlens_q), N.ptr(ctx.seq_start), None) if portions
            else (None, None, N.ptr(ctx.positions_i32)))
    return geom, ctx.batch_mapping.numel(), (int(ctx.max_seqlen_q) if portions else 1)


class DeltaRuleMixer(nn.Module):
    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, eps: float):
        super().__init__()
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        assert self.heads % self.kv_heads == 0
        self.taps, self.eps = int(conv), float(eps)
        G, D, H, Dv = self.kv_heads, self.dim, self.heads, self.vdim
        self.conv_channels = 2 * G * D + H * Dv
        # columns of the input projection, in this order
        self.in_parts: List[Tuple[str, int]] = [("q", G * D), ("k", G * D), ("v", H * Dv), ("g", H * Dv), ("b", H),
                                                ("a", H)]
        self.in_cols = sum(n for _, n in self.in_parts)
        self.in_bias = False
        f32 = dict(dtype=torch.float32)
        self.conv_weight = nn.Parameter(torch.empty(self.conv_channels, self.taps, **f32))
        self.A_log = nn.Parameter(torch.zeros(H, **f32))
        self.dt_bias = nn.Parameter(torch.zeros(H, **f32))
        self.norm_weight = nn.Parameter(torch.ones(Dv, **f32))
        self.o_proj = nn.Linear(H * Dv, width, bias=False)

    def make_state(self) -> MixerState:
        return MixerState({"conv_state": ((max(self.taps - 1, 1), self.conv_channels), None),
                           "matrix_state": ((self.heads, self.vdim, self.dim), torch.float32)})   # [value, key]

    def forward(self, h: torch.Tensor, cols: torch.Tensor, state: MixerState) -> torch.Tensor:
        """cols [T, in_cols] (row stride free): this mixer's columns of the projection of h."""
        ctx = get_context()
        assert state.matrix_state is not None, "state pool must be initialized"
        T = cols.shape[0]
        G, D, H, Dv = self.kv_heads, self.dim, self.heads, self.vdim
        dev, lib, st = cols.device, N.lib(), N.stream(cols.device)
        code = N.block_dtype_code(cols.dtype)
        assert cols.stride(1) == 1 and cols.shape[1] == self.in_cols and state.conv_state.dtype == cols.dtype
        geom, B, max_new = _geometry(ctx)
        slots = ctx.batch_mapping
        C = self.conv_channels
        qkv = torch.empty((T, C), dtype=torch.float32, device=dev)
        N.check(lib.cvllm_causal_conv(N.ptr(cols), cols.stride(0), 0, C, self.taps, N.ptr(self.conv_weight), None,
                                      N.ptr(state.conv_state), *geom, N.ptr(slots), B, max_new, N.ptr(qkv),
                                      qkv.stride(0), code, st), "cvllm_causal_conv")
        N.check(lib.cvllm_conv_state_update(N.ptr(cols), cols.stride(0), 0, C, self.taps, N.ptr(state.conv_state),
                                            *geom, N.ptr(slots), B, RESERVED_BATCH, code, st),
                "cvllm_conv_state_update")
        out = torch.empty((T, H * Dv), dtype=cols.dtype, device=dev)
        g_off = C
        b_off = C + H * Dv
        N.check(lib.cvllm_delta_rule(N.ptr(qkv), qkv.stride(0), N.ptr(cols), cols.stride(0), b_off, b_off + H,
                                     N.ptr(self.A_log), N.ptr(self.dt_bias), N.ptr(state.matrix_state), N.ptr(cols),
                                     cols.stride(0), g_off, N.ptr(self.norm_weight), 0, self.eps, *geom, N.ptr(slots),
                                     B, max_new, N.ptr(out), out.stride(0), H, G, D, Dv, RESERVED_BATCH, code, st),
                "cvllm_delta_rule")
        return self.o_proj(out)


class WkvMixer(nn.Module):
    BLENDS = ("r", "k", "v", "g", "w")

    def __init__(self, width: int, heads: int, dim: int, decay_rank: int, eps: float, dtype=None):
        super().__init__()
        self.width, self.heads, self.dim, self.eps = int(width), int(heads), int(dim), float(eps)
        HD = self.heads * self.dim
        self.in_parts: List[Tuple[str, int]] = []     # nothing of it reads the layer's input directly
        self.in_cols, self.in_bias = 0, False
        f32 = dict(dtype=torch.float32)
        self.mu = nn.Parameter(torch.zeros(len(self.BLENDS), width, **f32))
        self.rkvg = nn.Parameter(torch.empty(4, HD, width, dtype=dtype))     # r, k, v, gate projections
        self.w1 = nn.Linear(width, int(decay_rank), bias=False)
        self.w2 = nn.Linear(int(decay_rank), HD, bias=False)
        self.w0 = nn.Parameter(torch.zeros(HD, **f32))
        self.bonus = nn.Parameter(torch.zeros(HD, **f32))
        self.norm_weight = nn.Parameter(torch.ones(HD, **f32))
        self.o_proj = nn.Linear(HD, width, bias=False)

    def make_state(self) -> MixerState:
        return MixerState({"shift_state": ((self.width,), None),
                           "matrix_state": ((self.heads, self.dim, self.dim), torch.float32)})    # [value, key]

    def forward(self, h: torch.Tensor, cols: Optional[torch.Tensor], state: MixerState) -> torch.Tensor:
        ctx = get_context()
        assert state.matrix_state is not None, "state pool must be initialized"
        T, W = h.shape
        H, D = self.heads, self.dim
        HD = H * D
        dev, lib, st = h.device, N.lib(), N.stream(h.device)
        code = N.block_dtype_code(h.dtype)
        assert h.stride(1) == 1 and state.shift_state.dtype == h.dtype
        geom, B, max_new = _geometry(ctx)
        slots = ctx.batch_mapping
        S = len(self.BLENDS)
        blends = torch.empty((S, T, W), dtype=h.dtype, device=dev)
        N.check(lib.cvllm_token_shift_mix(N.ptr(h), h.stride(0), N.ptr(self.mu), S, W, N.ptr(state.shift_state), *geom,
                                          N.ptr(slots), B, max_new, N.ptr(blends), T, RESERVED_BATCH, code, st),
                "cvllm_token_shift_mix")
        rkvg = torch.bmm(blends[:4], self.rkvg.transpose(1, 2))                 # [4, T, HD]
        w_raw = self.w2(torch.tanh_(self.w1(blends[4])))                         # [T, HD] decay logits before w0
        out = torch.empty((T, HD), dtype=h.dtype, device=dev)
        N.check(lib.cvllm_wkv_scan(N.ptr(rkvg[0]), HD, N.ptr(rkvg[1]), HD, N.ptr(rkvg[2]), HD, N.ptr(w_raw),
                                   w_raw.stride(0), N.ptr(self.w0), N.ptr(self.bonus), N.ptr(state.matrix_state),
                                   N.ptr(rkvg[3]), HD, 0, N.ptr(self.norm_weight), D, self.eps, *geom, N.ptr(slots), B,
                                   max_new, N.ptr(out), out.stride(0), H, D, RESERVED_BATCH, code, st),
                "cvllm_wkv_scan")
        return self.o_proj(out)


GATE_SILU, GATE_SIGMOID = 0, 1


class GeneralDeltaMixer(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, decay_rank: int, rate: float, eps: float):
        super().__init__()
        self.width, self.heads, self.dim = int(width), int(heads), int(dim)
        self.rate, self.eps = float(rate), float(eps)
        HD = self.heads * self.dim
        self.in_parts: List[Tuple[str, int]] = [("r", HD), ("k", HD), ("v", HD), ("g", HD), ("a", HD),
                                                ("w1", int(decay_rank))]
        self.in_bias = True          # on the removal-rate columns only
        f32 = dict(dtype=torch.float32)
        self.w2 = nn.Linear(int(decay_rank), HD, bias=False)
        self.w0 = nn.Parameter(torch.zeros(HD, **f32))
        self.norm_weight = nn.Parameter(torch.ones(HD, **f32))
        self.o_proj = nn.Linear(HD, width, bias=False)

    @property
    def in_cols(self) -> int:
        return sum(n for _, n in self.in_parts)

    def set_decay_rank(self, rank: int) -> None:
        """The inner size of the decay projection comes with a checkpoint's tensors."""
        HD = self.heads * self.dim
        self.in_parts[-1] = ("w1", int(rank))
        self.w2 = nn.Linear(int(rank), HD, bias=False, device=self.w2.weight.device, dtype=self.w2.weight.dtype)

    def make_state(self) -> MixerState:
        return MixerState({"matrix_state": ((self.heads, self.dim, self.dim), torch.float32)})    # [value, key]

    def forward(self, h: torch.Tensor, cols: torch.Tensor, state: MixerState) -> torch.Tensor:
        """cols [T, in_cols] (row stride free): this mixer's columns of the projection of its input."""
        ctx = get_context()
        assert state.matrix_state is not None, "state pool must be initialized"
        T = cols.shape[0]
        H, D = self.heads, self.dim
        HD = H * D
        dev, lib, st = cols.device, N.lib(), N.stream(cols.device)
        code = N.block_dtype_code(cols.dtype)
        assert cols.stride(1) == 1 and cols.shape[1] == self.in_cols
        geom, B, max_new = _geometry(ctx)
        w_raw = self.w2(torch.tanh(cols[:, 5 * HD:]))                            # [T, HD] decay logits before w0
        out = torch.empty((T, HD), dtype=cols.dtype, device=dev)
        N.check(lib.cvllm_general_delta(N.ptr(cols), cols.stride(0), 0, HD, 2 * HD, 4 * HD, N.ptr(w_raw),
                                        w_raw.stride(0), N.ptr(self.w0), self.rate, N.ptr(state.matrix_state), 3 * HD,
                                        GATE_SIGMOID, N.ptr(self.norm_weight), D, self.eps, *geom,
                                        N.ptr(ctx.batch_mapping), B, max_new, N.ptr(out), out.stride(0), H, D,
                                        RESERVED_BATCH, code, st), "cvllm_general_delta")
        return self.o_proj(out)


class MatrixMemoryMixer(nn.Module):
    def __init__(self, width: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float):
        super().__init__()
        self.heads, self.dim, self.vdim = int(heads), int(dim), int(vdim)
        self.cap, self.eps = float(gate_cap), float(eps)
        H, D, Dv = self.heads, self.dim, self.vdim
        self.in_parts: List[Tuple[str, int]] = [("q", H * D), ("k", H * D), ("v", H * Dv), ("g", H * Dv), ("i", H),
                                                ("f", H)]
        self.in_cols = sum(n for _, n in self.in_parts)
        self.norm_weight = nn.Parameter(torch.ones(H * Dv, dtype=torch.float32))
        self.o_proj = nn.Linear(H * Dv, width, bias=False)

    def make_state(self) -> MixerState:
        f32 = torch.float32
        return MixerState({"matrix_state": ((self.heads, self.vdim, self.dim), f32),      # [value, key]
                           "norm_state": ((self.heads, self.dim), f32), "max_state": ((self.heads,), f32)})

    def forward(self, cols: torch.Tensor, state: MixerState) -> torch.Tensor:
        """cols [T, in_cols] (row stride free) -> W_o of the gated, normed read-out."""
        ctx = get_context()
        assert state.matrix_state is not None, "state pool must be initialized"
        T = cols.shape[0]
        H, D, Dv = self.heads, self.dim, self.vdim
        dev, lib, st = cols.device, N.lib(), N.stream(cols.device)
        code = N.block_dtype_code(cols.dtype)
        assert cols.stride(1) == 1 and cols.shape[1] == self.in_cols
        geom, B, max_new = _geometry(ctx)
        out = torch.empty((T, H * Dv), dtype=cols.dtype, device=dev)
        v_off = 2 * H * D
        g_off = v_off + H * Dv
        i_off = g_off + H * Dv
        N.check(lib.cvllm_matrix_memory(N.ptr(cols), cols.stride(0), 0, H * D, v_off, i_off, i_off + H, self.cap,
                                        D ** -0.5, N.ptr(state.matrix_state), N.ptr(state.norm_state),
                                        N.ptr(state.max_state), g_off, GATE_SIGMOID, N.ptr(self.norm_weight), Dv,
                                        self.eps, *geom, N.ptr(ctx.batch_mapping), B, max_new, N.ptr(out),
                                        out.stride(0), H, D, Dv, RESERVED_BATCH, code, st), "cvllm_matrix_memory")
        return self.o_proj(out)
