"""RMSNorm (reference: layers/layernorm.py:5-49) on the native kernel `cvllm_rmsnorm`.

Same module surface: `RMSNorm(hidden_size, eps).forward(x, residual=None)` returns the normed
tensor, or `(normed, new_residual)` when a residual is given.  The reference's two torch.compile'd
functions become one CTA-per-row launch with the reference's rounding points
(x.float() * rsqrt(mean + eps) -> model dtype -> * weight).  No CPU / eager fallback.
"""
from __future__ import annotations

import torch
from torch import nn

from compactor_vllm import _native as N


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """x [..., width] (last dim contiguous, rows uniformly strided); residual is updated IN PLACE
    like the reference's add_rms_forward result (it returns the new residual)."""
    width = x.shape[-1]
    x2 = x.reshape(-1, width)
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    o2 = out.view(-1, width)
    r2 = None
    if residual is not None:
        assert residual.shape == x.shape and residual.dtype == x.dtype
        r2 = residual.view(-1, width)
    w = weight if weight.dtype == x.dtype else weight.to(x.dtype)
    assert x2.stride(-1) == 1 and w.is_contiguous()
    rc = N.lib().cvllm_rmsnorm(
        N.ptr(x2), N.ptr(r2), N.ptr(w), N.ptr(o2), x2.stride(0), r2.stride(0) if r2 is not None else 0,
        o2.stride(0), x2.shape[0], width, float(eps), N.dtype_code(x.dtype), N.stream(x.device),
    )
    N.check(rc, "cvllm_rmsnorm")
    return out if residual is None else (out, residual)


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def rms_forward(self, x: torch.Tensor) -> torch.Tensor:
        return rms_norm(x, self.weight, self.eps)

    def add_rms_forward(self, x: torch.Tensor, residual: torch.Tensor):
        return rms_norm(x, self.weight, self.eps, residual)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        if residual is None:
            return self.rms_forward(x)
        return self.add_rms_forward(x, residual)


def sandwich_norm(resid: torch.Tensor, *, branch: torch.Tensor | None = None, post_weight: torch.Tensor | None = None,
                  pre_weight: torch.Tensor | None = None, eps: float = 1e-6, out_dtype: torch.dtype | None = None,
                  gain_offset: float = 0.0, assign: bool = False, cast_out: bool = False):
    """One launch of `cvllm_sandwich_norm` on a 32-bit residual stream `resid` [T, width], updated IN PLACE:

        branch given:      resid += branch / sqrt(mean(branch^2) + eps) * (post_weight + gain_offset)
                           (`assign`: resid = that, without the sum - the norm of an embedding that starts the stream)
        pre_weight given:  returns  resid / sqrt(mean(resid^2) + eps) * (pre_weight + gain_offset)  in `out_dtype`
        cast_out:          returns  resid itself rounded to `out_dtype` (models whose sublayers read the stream unnormed)

    i.e. the post-norm of one sublayer's output, the residual sum and the pre-norm of the next sublayer.  Statistics,
    sum and residual are fp32 whatever the activations' dtype; the weights are fp32 tensors (`gain_offset` 1 for
    gains stored around zero)."""
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.stride(1) == 1
    rows, width = resid.shape
    y_code = o_code = N.CVLLM_F32
    y_stride = o_stride = 0
    out = None
    if branch is not None:
        assert branch.shape == resid.shape and branch.stride(1) == 1 and post_weight.dtype == torch.float32
        y_code, y_stride = N.block_dtype_code(branch.dtype), branch.stride(0)
    assert pre_weight is None or not cast_out
    if pre_weight is not None or cast_out:
        assert pre_weight is None or pre_weight.dtype == torch.float32
        out = torch.empty((rows, width), dtype=out_dtype or torch.float32, device=resid.device)
        o_code, o_stride = N.block_dtype_code(out.dtype), out.stride(0)
    rc = N.lib().cvllm_sandwich_norm(
        N.ptr(branch), y_stride, y_code, N.ptr(post_weight) if branch is not None else None, N.ptr(resid),
        resid.stride(0), N.ptr(pre_weight), N.ptr(out), o_stride, o_code, rows, width, float(eps), float(gain_offset),
        int(bool(assign)), N.stream(resid.device))
    N.check(rc, "cvllm_sandwich_norm")
    return out


class NormWeight(nn.Module):
    """An RMS-norm gain kept in fp32 whatever the model dtype (the norm itself runs inside `sandwich_norm`)."""

    def __init__(self, size: int) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size, dtype=torch.float32))


NORM_RMS, NORM_LAYER = 0, 1


def residual_norm(resid: torch.Tensor, *, add: tuple = (), add_f32: torch.Tensor | None = None,
                  weight: torch.Tensor | None = None, bias: torch.Tensor | None = None, eps: float = 1e-6,
                  kind: int = NORM_LAYER, out_dtype: torch.dtype | None = None):
    """One launch of `cvllm_residual_norm` on a 32-bit residual stream `resid` [T, width], updated IN PLACE:

        resid += add[0] + add[1] + add_f32      (up to two branch outputs in the activations' type, one fp32 tensor)
        weight given:  returns norm(resid) in `out_dtype` - NORM_LAYER: (x - mean) / sqrt(var + eps) * weight + bias,
                       NORM_RMS: x / sqrt(mean(x^2) + eps) * weight

    i.e. the residual sum of a layer whose sublayers run side by side on one normed input, fused with the norm in
    front of the next layer.  Sum and statistics are fp32; weight and bias are fp32 tensors."""
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.stride(1) == 1
    rows, width = resid.shape
    add = tuple(t for t in add if t is not None)
    assert len(add) <= 2
    a = add[0] if len(add) > 0 else None
    b = add[1] if len(add) > 1 else None
    ab_code = N.CVLLM_F32
    for t in add:
        assert t.shape == resid.shape and t.stride(1) == 1 and t.dtype == add[0].dtype
        ab_code = N.block_dtype_code(t.dtype)
    if add_f32 is not None:
        assert add_f32.shape == resid.shape and add_f32.dtype == torch.float32 and add_f32.stride(1) == 1
    out, o_code, o_stride = None, N.CVLLM_F32, 0
    if weight is not None:
        assert weight.dtype == torch.float32 and (bias is None or bias.dtype == torch.float32)
        out = torch.empty((rows, width), dtype=out_dtype or torch.float32, device=resid.device)
        o_code, o_stride = N.block_dtype_code(out.dtype), out.stride(0)
    rc = N.lib().cvllm_residual_norm(
        N.ptr(a), a.stride(0) if a is not None else 0, N.ptr(b), b.stride(0) if b is not None else 0, ab_code,
        N.ptr(add_f32), add_f32.stride(0) if add_f32 is not None else 0, N.ptr(resid), resid.stride(0), N.ptr(weight),
        N.ptr(bias), N.ptr(out), o_stride, o_code, rows, width, float(eps), int(kind), N.stream(resid.device))
    N.check(rc, "cvllm_residual_norm")
    return out


def gated_residual_norm(resid: torch.Tensor, *, branch: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                        weight: torch.Tensor | None = None, eps: float = 1e-6, out_dtype: torch.dtype | None = None):
    """One launch of `cvllm_gated_residual_norm` on a 32-bit residual stream `resid` [T, width], updated IN PLACE:

        branch given:  resid += sigmoid(gate) * branch     (gate logits and branch [T, width], bfloat16 or float32)
        weight given:  returns resid / sqrt(mean(resid^2) + eps) * weight in `out_dtype`

    i.e. the gated residual sum of one sublayer fused with the RMS norm in front of the next."""
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.stride(1) == 1
    rows, width = resid.shape
    y_code = g_code = o_code = N.CVLLM_F32
    y_stride = g_stride = o_stride = 0
    if branch is not None:
        assert gate is not None and branch.shape == resid.shape == gate.shape
        assert branch.stride(1) == 1 and gate.stride(1) == 1
        y_code, y_stride = N.block_dtype_code(branch.dtype), branch.stride(0)
        g_code, g_stride = N.block_dtype_code(gate.dtype), gate.stride(0)
    out = None
    if weight is not None:
        assert weight.dtype == torch.float32
        out = torch.empty((rows, width), dtype=out_dtype or torch.float32, device=resid.device)
        o_code, o_stride = N.block_dtype_code(out.dtype), out.stride(0)
    rc = N.lib().cvllm_gated_residual_norm(
        N.ptr(branch), y_stride, y_code, N.ptr(gate) if branch is not None else None, g_stride, g_code, N.ptr(resid),
        resid.stride(0), N.ptr(weight), N.ptr(out), o_stride, o_code, rows, width, float(eps), N.stream(resid.device))
    N.check(rc, "cvllm_gated_residual_norm")
    return out


def dual_norm_blend(a: torch.Tensor, wa: torch.Tensor, b: torch.Tensor, wb: torch.Tensor, eps: float,
                    scale: float = 0.5) -> torch.Tensor:
    """scale * (rms_norm(a) * wa + rms_norm(b) * wb) per row (`cvllm_dual_norm_blend`): two branch outputs, each
    RMS-normed with a weight of its own, blended; fp32 inside, the result in the branches' type."""
    assert a.shape == b.shape and a.dtype == b.dtype and a.stride(1) == 1 and b.stride(1) == 1
    assert wa.dtype == torch.float32 and wb.dtype == torch.float32
    rows, width = a.shape
    out = torch.empty((rows, width), dtype=a.dtype, device=a.device)
    rc = N.lib().cvllm_dual_norm_blend(N.ptr(a), a.stride(0), N.ptr(wa), N.ptr(b), b.stride(0), N.ptr(wb), N.ptr(out),
                                       out.stride(0), rows, width, float(eps), float(scale),
                                       N.block_dtype_code(a.dtype), N.stream(a.device))
    N.check(rc, "cvllm_dual_norm_blend")
    return out


class LayerNormWeight(nn.Module):
    """Gain and bias of a layer norm kept in fp32 whatever the model dtype (the norm runs inside `residual_norm`)."""

    def __init__(self, size: int) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(size, dtype=torch.float32))
        self.bias = nn.Parameter(torch.zeros(size, dtype=torch.float32))
