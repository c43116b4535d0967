"""Feed-forward blocks: a gated dense layer and a routed mixture of experts.

Matrix products are library GEMMs (`torch.nn.functional.linear`), as in the other models; the gated activation,
the router's choice and the weighted combine are kernels of the native library (csrc/blocks.cu).
"""
from __future__ import annotations

import warnings

import torch
import torch.nn.functional as F
from torch import nn

from compactor_vllm import _native as N
from compactor_vllm.utils.context import get_context

ACT_SILU, ACT_GELU_TANH, ACT_CLAMPED_GLU = 0, 1, 2
ROUTE_SOFTMAX_ALL, ROUTE_TOP_LOGITS, ROUTE_SIGMOID = 0, 1, 2
ACT_RELU_SQUARED = 0      # kinds of `unary_act`


def gated_act(x: torch.Tensor, kind: int, rows: int | None = None, limit: float = 0.0) -> torch.Tensor:
    """x [T, 2F] = [gate | up] -> [T, F] (fp32 inside).  kind ACT_SILU / ACT_GELU_TANH: act(gate) * up;
    ACT_CLAMPED_GLU: g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1).
    `rows`: only the first so many rows are computed (the output still has T rows)."""
    T, F2 = x.shape
    assert F2 % 2 == 0 and x.stride(1) == 1
    out = torch.empty((T, F2 // 2), dtype=x.dtype, device=x.device)
    rc = N.lib().cvllm_gated_act(N.ptr(x), x.stride(0), N.ptr(out), out.stride(0), T if rows is None else int(rows),
                                 F2 // 2, int(kind), float(limit), N.block_dtype_code(x.dtype), N.stream(x.device))
    N.check(rc, "cvllm_gated_act")
    return out


def route(logits: torch.Tensor, correction: torch.Tensor | None, top: int, groups: int, keep: int,
          mode: int = ROUTE_SOFTMAX_ALL, experts: int | None = None):
    """fp32 router logits [T, E] -> (idx int32 [T, top], weights fp32 [T, top]).

    ROUTE_SOFTMAX_ALL: s = softmax(logits); the choice is made on s + correction among the experts of the `keep` best
    of `groups` neighbour groups (a group's rank is its largest s + correction); the weights are the chosen experts'
    plain s.  ROUTE_TOP_LOGITS: the `top` largest logits are chosen, the weights are the softmax over those alone.
    ROUTE_SIGMOID: the `top` largest sigmoid(logit) are chosen, each with its own sigmoid as weight (not renormalized).
    `experts`: only the first so many columns are router outputs (the rows may carry more, e.g. a gate logit)."""
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    T, E = logits.shape
    E = E if experts is None else int(experts)
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    wts = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    rc = N.lib().cvllm_moe_route(N.ptr(logits), logits.stride(0), N.ptr(correction), T, E, int(top), int(groups),
                                 int(keep), int(mode), N.ptr(idx), N.ptr(wts), N.stream(logits.device))
    N.check(rc, "cvllm_moe_route")
    return idx, wts


def unary_act(x: torch.Tensor, kind: int = ACT_RELU_SQUARED) -> torch.Tensor:
    """x [T, F] (row stride free) -> act(x) [T, F] (fp32 inside).  ACT_RELU_SQUARED: relu(x) ** 2."""
    T, F_ = x.shape
    assert x.stride(1) == 1
    out = torch.empty((T, F_), dtype=x.dtype, device=x.device)
    N.check(N.lib().cvllm_unary_act(N.ptr(x), x.stride(0), N.ptr(out), out.stride(0), T, F_, int(kind),
                                    N.block_dtype_code(x.dtype), N.stream(x.device)), "cvllm_unary_act")
    return out


class PlainMLP(nn.Module):
    """down(act(up x + b) ) + b: an ungated feed-forward with biases; act = relu squared."""

    def __init__(self, width: int, ff: int, act: int = ACT_RELU_SQUARED):
        super().__init__()
        self.act = act
        self.up_proj = nn.Linear(width, ff, bias=True)
        self.down_proj = nn.Linear(ff, width, bias=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(unary_act(self.up_proj(x), self.act))


class GatedMLP(nn.Module):
    """down(act(gate x) * up x), gate and up packed in one GEMM (`limit`: the clamp of ACT_CLAMPED_GLU)."""

    def __init__(self, width: int, ff: int, act: int, limit: float = 0.0):
        super().__init__()
        self.act, self.limit = act, float(limit)
        self.gate_up_proj = nn.Linear(width, 2 * ff, bias=False)
        self.down_proj = nn.Linear(ff, width, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(gated_act(self.gate_up_proj(x), self.act, limit=self.limit))


class RoutedExperts(nn.Module):
    """Mixture of `experts` gated experts and `identity` experts that return their input, `top` per token, with
    group-limited choice, a correction that shifts the choice but not the weights, and an optional shared expert.
    Options: `route_mode` ROUTE_TOP_LOGITS (choice on the logits, softmax over the chosen), `router_bias` (a bias on
    the logits), `limit` / `shared_limit` (clamps of ACT_CLAMPED_GLU), `shared_gate` (the shared expert's output is
    multiplied by the sigmoid of one more router row, so `router` has a row more than there are experts),
    `route_mode` ROUTE_SIGMOID (see `route`), `scale_inputs` (the routing weight multiplies the expert's INPUT, rounded
    to the activations' type, instead of its output: the outputs are summed unweighted).

    The router runs in fp32.  Portions: (token, choice) pairs are sorted by expert; in bfloat16 (sizes multiples of 8)
    the two projections are library grouped GEMMs over the segments (`torch._grouped_mm`, segment ends on the device);
    otherwise - float32, odd sizes - each expert with tokens runs its two GEMMs on its segment and the per-expert
    counts cross to the host once per layer.  Few tokens (decode steps, and any step of
    at most `SMALL_STEP` tokens): `cvllm_expert_gemv` reads each chosen expert's rows straight from the routing
    indices on the device, so the step has no host round trip and can be captured in a CUDA graph.  Either way the
    combine kernel sums the `top` outputs of every token (identity experts and the shared expert included) in fp32.
    Returns fp32 [T, width]."""

    SMALL_STEP = 8
    grouped_gemm = hasattr(torch, "_grouped_mm")     # False: the per-expert loop also in bfloat16 (tests compare them)

    def __init__(self, width: int, ff: int, experts: int, identity: int, top: int, groups: int, keep: int,
                 shared_ff: int, act: int = ACT_SILU, dtype: torch.dtype | None = None, *,
                 route_mode: int = ROUTE_SOFTMAX_ALL, router_bias: bool = False, limit: float = 0.0,
                 shared_limit: float = 0.0, shared_gate: bool = False, scale_inputs: bool = False):
        super().__init__()
        self.scale_inputs = bool(scale_inputs)
        assert not (scale_inputs and identity), "identity experts have no input to scale"
        self.width, self.ff, self.n_real, self.n_identity = width, ff, experts, identity
        self.top, self.groups, self.keep, self.act = top, groups, keep, act
        self.route_mode, self.limit = int(route_mode), float(limit)
        self.total = total = experts + identity
        self.shared_gate = bool(shared_gate and shared_ff)
        rows = total + (1 if self.shared_gate else 0)      # the last row: the shared expert's gate logit
        self.router = nn.Parameter(torch.empty(rows, width, dtype=torch.float32))
        self.router_bias = nn.Parameter(torch.zeros(rows, dtype=torch.float32)) if router_bias else None
        self.correction = (nn.Parameter(torch.zeros(total, dtype=torch.float32))
                           if route_mode == ROUTE_SOFTMAX_ALL else None)
        self.gate_up = nn.Parameter(torch.empty(experts, 2 * ff, width, dtype=dtype))
        self.down = nn.Parameter(torch.empty(experts, width, ff, dtype=dtype))
        self.shared = GatedMLP(width, shared_ff, act, shared_limit) if shared_ff else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        T, W = x.shape
        logits = F.linear(x.float(), self.router, self.router_bias)
        idx, wts = route(logits, self.correction, self.top, self.groups, self.keep, self.route_mode, self.total)
        shared = self.shared(x) if self.shared is not None else None
        gate = (N.ptr(logits) + 4 * self.total, logits.stride(0)) if self.shared_gate else (None, 0)
        out = torch.empty((T, W), dtype=torch.float32, device=x.device)
        lib, code, st = N.lib(), N.block_dtype_code(x.dtype), N.stream(x.device)
        cw = None if self.scale_inputs else N.ptr(wts)     # weights of the combine (None: all 1)

        def scaled(perm):     # rows of the pairs (in `perm`'s order), each times its routing weight
            rows = torch.empty((T * self.top, W), dtype=x.dtype, device=x.device)
            N.check(lib.cvllm_scaled_rows(N.ptr(x), x.stride(0), N.ptr(perm), N.ptr(wts), self.top, N.ptr(rows),
                                          T * self.top, W, code, st), "cvllm_scaled_rows")
            return rows

        if not get_context().is_prefill or T <= self.SMALL_STEP:
            pairs = T * self.top
            a = torch.empty((pairs, self.ff), dtype=x.dtype, device=x.device)
            ys = torch.empty((pairs, W), dtype=x.dtype, device=x.device)
            src, div = (scaled(None), 1) if self.scale_inputs else (x, self.top)
            N.check(lib.cvllm_expert_gemv(N.ptr(src), div, N.ptr(self.gate_up), N.ptr(idx), self.n_real, N.ptr(a),
                                          pairs, self.ff, W, self.act, self.limit, code, st), "cvllm_expert_gemv")
            N.check(lib.cvllm_expert_gemv(N.ptr(a), 1, N.ptr(self.down), N.ptr(idx), self.n_real, N.ptr(ys),
                                          pairs, W, self.ff, -1, 0.0, code, st), "cvllm_expert_gemv")
            N.check(lib.cvllm_moe_combine(N.ptr(ys), None, cw, self.top, N.ptr(idx), self.n_real, N.ptr(x),
                                          N.ptr(shared), *gate, N.ptr(out), T, W, code, st), "cvllm_moe_combine")
            return out
        # pairs sorted by expert (identity experts' pairs come last and are never multiplied); every buffer has
        # T * top rows whatever the routing, so the allocator sees the same sizes every step
        flat = idx.view(-1).long()
        order = torch.argsort(flat, stable=True)
        pos = torch.empty_like(order, dtype=torch.int32)
        pos[order] = torch.arange(order.numel(), dtype=torch.int32, device=x.device)
        xs = scaled(order) if self.scale_inputs else x.index_select(0, order // self.top)
        counts = torch.zeros(self.n_real + self.n_identity, dtype=torch.int32, device=x.device)
        counts.index_add_(0, flat, torch.ones_like(flat, dtype=torch.int32))
        ys = None
        if self.grouped_gemm and x.dtype == torch.bfloat16 and W % 8 == 0 and self.ff % 8 == 0:
            # library grouped GEMM: segment ends stay on the device, one launch per projection, no host round trip
            # and no per-shape algorithm search (a plain GEMM with a row count it has not seen costs milliseconds)
            ends = counts[: self.n_real].cumsum(0).to(torch.int32)
            try:
                gu = torch._grouped_mm(xs, self.gate_up.transpose(1, 2), offs=ends)
                ys = torch._grouped_mm(gated_act(gu, self.act, limit=self.limit), self.down.transpose(1, 2), offs=ends)
            except (RuntimeError, NotImplementedError) as ex:   # a shape the library's grouped kernel refuses
                warnings.warn(f"grouped GEMM refused ({ex}); the per-expert products serve this layer from now on")
                self.grouped_gemm = False
        if ys is None:
            host_counts = counts[: self.n_real].tolist()
            gu = torch.empty((order.numel(), 2 * self.ff), dtype=x.dtype, device=x.device)
            ys = torch.empty((order.numel(), W), dtype=x.dtype, device=x.device)
            off = 0
            for e, c in enumerate(host_counts):
                if c:
                    torch.mm(xs[off:off + c], self.gate_up[e].t(), out=gu[off:off + c])
                    off += c
            a = gated_act(gu, self.act, rows=off, limit=self.limit)
            off = 0
            for e, c in enumerate(host_counts):
                if c:
                    torch.mm(a[off:off + c], self.down[e].t(), out=ys[off:off + c])
                    off += c
        N.check(lib.cvllm_moe_combine(N.ptr(ys), N.ptr(pos), cw, self.top, N.ptr(idx), self.n_real, N.ptr(x),
                                      N.ptr(shared), *gate, N.ptr(out), T, W, code, st), "cvllm_moe_combine")
        return out
