"""State-space mixer with a scalar decay per head (the multi-head "state-space duality" form).

From its input h the layer projects  [z | x | B | C | dt] = W_in h  (z, x: heads * vdim; B, C: groups * state; dt: heads),
passes x, B and C through a causal convolution per channel with silu, and runs per head h (group g = h // (heads / groups))
    dt_t = softplus(dt_t + dt_bias_h)       S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t x_t B_t^T       y_t = S_t C_t + D_h x_t
then  out = W_o (unit_norm_per_part(y * silu(z)) * w).  The recurrence, its decay, the step size, the gate and the norm
are fp32; S [heads, vdim, state] fp32 and the convolution's last taps - 1 inputs are the sequence's state, kept in the
slot of a state pool (kv_cache/state_pool.py) between steps.  A step may bring any number of tokens per sequence; a
portion that starts at position 0 starts from a zero state.  Kernels: csrc/ssm.cu.

`SelectiveScanMixer` is the older form with a decay per (channel, state channel): [x | z] = W_in h, x through the causal
convolution (with bias) and silu, [dt | B | C] = W_x x, dt = softplus(W_dt dt + b) per channel, A = -exp(A_log),
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n        y_c = sum_n S[c, n] C_n + D_c x_c
then  out = W_o (y * silu(z)).  `ResidualShortConv` is the convolution alone, added to its own input.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from compactor_vllm import _native as N
from compactor_vllm.config.constants import RESERVED_BATCH
from compactor_vllm.utils.context import get_context


class StateSpaceMixer(nn.Module):
    def __init__(self, width: int, heads: int, vdim: int, state: int, groups: int, conv: int, norm_groups: int,
                 eps: float):
        super().__init__()
        self.heads, self.vdim, self.state, self.groups = int(heads), int(vdim), int(state), int(groups)
        self.taps, self.norm_groups, self.eps = int(conv), int(norm_groups), float(eps)
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.state
        self.in_proj = nn.Linear(width, 2 * self.inner + 2 * self.groups * self.state + self.heads, bias=False)
        f32 = dict(dtype=torch.float32)
        self.conv_weight = nn.Parameter(torch.empty(self.channels, self.taps, **f32))
        self.conv_bias = nn.Parameter(torch.zeros(self.channels, **f32))
        self.dt_bias = nn.Parameter(torch.zeros(self.heads, **f32))
        self.A_log = nn.Parameter(torch.zeros(self.heads, **f32))
        self.D = nn.Parameter(torch.ones(self.heads, **f32))
        self.norm_weight = nn.Parameter(torch.ones(self.inner, **f32))
        self.o_proj = nn.Linear(self.inner, width, bias=False)
        # injected by the state pool: [slots, taps - 1, channels] (model dtype) and [slots, heads, vdim, state] fp32
        self.conv_state: Optional[torch.Tensor] = None
        self.ssm_state: Optional[torch.Tensor] = None

    def state_specs(self, dtype: torch.dtype):
        """name -> (shape per slot, dtype) of what a sequence carries from step to step."""
        return {"conv_state": ((max(self.taps - 1, 1), self.channels), dtype),
                "ssm_state": ((self.heads, self.vdim, self.state), torch.float32)}

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        ctx = get_context()
        assert self.ssm_state is not None, "state pool must be initialized"
        T = h.shape[0]
        dev, lib, st = h.device, N.lib(), N.stream(h.device)
        proj = self.in_proj(h)
        code = N.block_dtype_code(proj.dtype)
        assert self.conv_state.dtype == proj.dtype
        portions = ctx.is_prefill      # else: one token per sequence, at positions_i32
        geom = ((N.ptr(ctx.cu_seqlens_q), N.ptr(ctx.seq_start), None) if portions
                else (None, None, N.ptr(ctx.positions_i32)))
        slots = ctx.batch_mapping
        B = slots.numel()
        max_new = int(ctx.max_seqlen_q) if portions else 1
        xbc = torch.empty((T, self.channels), dtype=torch.float32, device=dev)
        N.check(lib.cvllm_causal_conv(N.ptr(proj), proj.stride(0), self.inner, self.channels, self.taps,
                                      N.ptr(self.conv_weight), N.ptr(self.conv_bias), N.ptr(self.conv_state), *geom,
                                      N.ptr(slots), B, max_new, N.ptr(xbc), xbc.stride(0), code, st), "cvllm_causal_conv")
        N.check(lib.cvllm_conv_state_update(N.ptr(proj), proj.stride(0), self.inner, self.channels, self.taps,
                                            N.ptr(self.conv_state), *geom, N.ptr(slots), B, RESERVED_BATCH, code, st),
                "cvllm_conv_state_update")
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        ws_bytes = lib.cvllm_ssm_scan_workspace_bytes(B, max_new, self.heads, self.vdim, self.state)
        ws = N.workspace(dev, ws_bytes, "ssm_scan") if ws_bytes else None     # long portions: per-segment states
        N.check(lib.cvllm_ssm_scan(N.ptr(xbc), xbc.stride(0), N.ptr(proj), proj.stride(0), self.inner + self.channels,
                                   N.ptr(self.dt_bias), N.ptr(self.A_log), N.ptr(self.D), N.ptr(self.ssm_state), *geom,
                                   N.ptr(slots), B, max_new, N.ptr(y), y.stride(0), self.heads, self.groups, self.vdim,
                                   self.state, RESERVED_BATCH, N.ptr(ws), ws_bytes, code, st), "cvllm_ssm_scan")
        out = torch.empty((T, self.inner), dtype=proj.dtype, device=dev)
        N.check(lib.cvllm_gated_group_norm(N.ptr(y), y.stride(0), N.ptr(proj), proj.stride(0), N.ptr(self.norm_weight),
                                           self.eps, N.ptr(out), out.stride(0), T, self.inner, self.norm_groups, code, st),
                "cvllm_gated_group_norm")
        return self.o_proj(out)


class ResidualShortConv(nn.Module):
    """out = h + causal_conv(h): a short convolution per channel over time (no bias, no activation) added to its own
    input; the last taps - 1 inputs of a sequence live in the state pool (`conv_state`)."""

    def __init__(self, channels: int, taps: int):
        super().__init__()
        self.channels, self.taps = int(channels), int(taps)
        self.weight = nn.Parameter(torch.zeros(self.channels, self.taps, dtype=torch.float32))
        self.conv_state: Optional[torch.Tensor] = None

    def state_specs(self, dtype: torch.dtype):
        return {"conv_state": ((max(self.taps - 1, 1), self.channels), dtype)}

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        ctx = get_context()
        assert self.conv_state is not None, "state pool must be initialized"
        assert h.stride(1) == 1 and h.shape[1] == self.channels and self.conv_state.dtype == h.dtype
        T = h.shape[0]
        dev, lib, st = h.device, N.lib(), N.stream(h.device)
        code = N.block_dtype_code(h.dtype)
        portions = ctx.is_prefill
        geom = ((N.ptr(ctx.cu_seqlens_q), N.ptr(ctx.seq_start), None) if portions
                else (None, None, N.ptr(ctx.positions_i32)))
        slots = ctx.batch_mapping
        B = slots.numel()
        max_new = int(ctx.max_seqlen_q) if portions else 1
        out = torch.empty((T, self.channels), dtype=h.dtype, device=dev)
        N.check(lib.cvllm_causal_conv_mode(N.ptr(h), h.stride(0), 0, self.channels, self.taps, N.ptr(self.weight), None,
                                           N.ptr(self.conv_state), *geom, N.ptr(slots), B, max_new, N.ptr(out),
                                           out.stride(0), code, 1, code, st), "cvllm_causal_conv_mode")
        N.check(lib.cvllm_conv_state_update(N.ptr(h), h.stride(0), 0, self.channels, self.taps, N.ptr(self.conv_state),
                                            *geom, N.ptr(slots), B, RESERVED_BATCH, code, st),
                "cvllm_conv_state_update")
        return out


class SelectiveScanMixer(nn.Module):
    def __init__(self, width: int, inner: int, state: int, dt_rank: int, conv: int):
        super().__init__()
        self.inner, self.state, self.dt_rank, self.taps = int(inner), int(state), int(dt_rank), int(conv)
        self.in_parts = [("in", 2 * self.inner)]       # [x | z]
        self.in_cols, self.in_bias = 2 * self.inner, False
        f32 = dict(dtype=torch.float32)
        self.conv_weight = nn.Parameter(torch.empty(self.inner, self.taps, **f32))
        self.conv_bias = nn.Parameter(torch.zeros(self.inner, **f32))
        self.x_proj = nn.Linear(self.inner, self.dt_rank + 2 * self.state, bias=False)
        self.dt_proj = nn.Linear(self.dt_rank, self.inner, bias=False)
        self.dt_bias = nn.Parameter(torch.zeros(self.inner, **f32))
        self.A_log = nn.Parameter(torch.zeros(self.inner, self.state, **f32))
        self.D = nn.Parameter(torch.ones(self.inner, **f32))
        self.o_proj = nn.Linear(self.inner, width, bias=False)
        self.conv_state: Optional[torch.Tensor] = None
        self.scan_state: Optional[torch.Tensor] = None

    def state_specs(self, dtype: torch.dtype):
        return {"conv_state": ((max(self.taps - 1, 1), self.inner), dtype),
                "scan_state": ((self.inner, self.state), torch.float32)}

    def forward(self, cols: torch.Tensor) -> torch.Tensor:
        """cols [T, 2 * inner] = [x | z] (row stride free): the projection of the mixer's input."""
        ctx = get_context()
        assert self.scan_state is not None, "state pool must be initialized"
        T = cols.shape[0]
        dev, lib, st = cols.device, N.lib(), N.stream(cols.device)
        code = N.block_dtype_code(cols.dtype)
        assert cols.stride(1) == 1 and cols.shape[1] == 2 * self.inner and self.conv_state.dtype == cols.dtype
        portions = ctx.is_prefill
        geom = ((N.ptr(ctx.cu_seqlens_q), N.ptr(ctx.seq_start), None) if portions
                else (None, None, N.ptr(ctx.positions_i32)))
        slots = ctx.batch_mapping
        B = slots.numel()
        max_new = int(ctx.max_seqlen_q) if portions else 1
        x = torch.empty((T, self.inner), dtype=cols.dtype, device=dev)
        N.check(lib.cvllm_causal_conv_mode(N.ptr(cols), cols.stride(0), 0, self.inner, self.taps,
                                           N.ptr(self.conv_weight), N.ptr(self.conv_bias), N.ptr(self.conv_state),
                                           *geom, N.ptr(slots), B, max_new, N.ptr(x), x.stride(0), code, 0, code, st),
                "cvllm_causal_conv_mode")
        N.check(lib.cvllm_conv_state_update(N.ptr(cols), cols.stride(0), 0, self.inner, self.taps,
                                            N.ptr(self.conv_state), *geom, N.ptr(slots), B, RESERVED_BATCH, code, st),
                "cvllm_conv_state_update")
        dbc = self.x_proj(x)                                       # [dt | B | C]
        dt_raw = self.dt_proj(dbc[:, :self.dt_rank])
        out = torch.empty((T, self.inner), dtype=cols.dtype, device=dev)
        R, S = self.dt_rank, self.state
        N.check(lib.cvllm_selective_scan(N.ptr(x), x.stride(0), N.ptr(dt_raw), dt_raw.stride(0), N.ptr(self.dt_bias),
                                         N.ptr(dbc), dbc.stride(0), R, R + S, N.ptr(self.A_log), N.ptr(self.D),
                                         N.ptr(cols), cols.stride(0), self.inner, N.ptr(self.scan_state), *geom,
                                         N.ptr(slots), B, max_new, N.ptr(out), out.stride(0), self.inner, S,
                                         RESERVED_BATCH, code, st), "cvllm_selective_scan")
        return self.o_proj(out)
