"""RMSNorm and add + RMSNorm on the fp32 residual stream: the step right before the q/k/v and
gate/up projections, which hands them their fp16 input.

Mirrors the reference's `rms_norm` / `add_rms_norm` (solution/rmsnorm.py:52-150; used by
solution/packed.py:88-115) without the host-offload option: one kernel pass per direction, the
only thing kept for the backward besides the normalised tensor is one fp32 number per row.
"""

from __future__ import annotations

import torch

from . import _lib
from .nf4 import _stream_ptr


def _check(x, weight):
    if not (x.is_cuda and weight.is_cuda):
        raise ValueError("hackaton_b200: RMSNorm needs CUDA tensors (there is no CPU path)")
    if x.dtype != torch.float32 or weight.dtype != torch.float32:
        raise TypeError(f"hackaton_b200: RMSNorm runs on the fp32 stream, got {x.dtype}, {weight.dtype}")
    if weight.numel() != x.shape[-1]:
        raise ValueError("hackaton_b200: RMSNorm weight does not match the last dimension")


def _forward(x2, delta2, weight, eps, to_half):
    rows, hidden = x2.shape
    out = torch.empty((rows, hidden), dtype=torch.float16 if to_half else torch.float32, device=x2.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x2.device)
    total = torch.empty_like(x2) if delta2 is not None else None
    with torch.cuda.device(x2.device):
        _lib.check(_lib.lib().nf4b200_rmsnorm_fwd(
            x2.data_ptr(), None if delta2 is None else delta2.data_ptr(), weight.data_ptr(),
            None if total is None else total.data_ptr(), out.data_ptr(),
            _lib.F16 if to_half else _lib.F32, rstd.data_ptr(), rows, hidden, float(eps),
            _stream_ptr(x2.device)))
    return out, rstd, total


def _backward(x2, weight, rstd, dy2, d_total):
    rows, hidden = x2.shape
    dx = torch.empty_like(x2)
    with torch.cuda.device(x2.device):
        _lib.check(_lib.lib().nf4b200_rmsnorm_bwd(
            x2.data_ptr(), weight.data_ptr(), rstd.data_ptr(), dy2.data_ptr(),
            _lib.F16 if dy2.dtype == torch.float16 else _lib.F32,
            None if d_total is None else d_total.data_ptr(), dx.data_ptr(), rows, hidden,
            _stream_ptr(x2.device)))
    return dx


def _dweight(dy2, x2, rstd, weight):
    """solution/rmsnorm.py:93-95: not on the task's path (frozen norm weights), plain torch."""
    return (dy2.float() * (x2 * rstd[:, None])).sum(dim=0).to(weight.dtype)


class RMSNorm(torch.autograd.Function):
    """weight * (x * rsqrt(mean(x^2) + eps)) for fp32 x (solution/rmsnorm.py:52-96)."""

    @staticmethod
    def forward(ctx, x, weight, eps, to_half=False):
        _check(x, weight)
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        weight = weight.contiguous()
        out, rstd, _ = _forward(x2, None, weight, eps, to_half)
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = shape
        return out.reshape(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, rstd = ctx.saved_tensors
        dy2 = dy.reshape(x2.shape).contiguous()
        dx = _backward(x2, weight, rstd, dy2, None)
        dweight = _dweight(dy2, x2, rstd, weight) if ctx.needs_input_grad[1] else None
        return dx.reshape(ctx.shape), dweight, None, None


def rms_norm(x, weight, eps, to_half=False):
    """solution/rmsnorm.py:99-101."""
    return RMSNorm.apply(x, weight, eps, to_half)


class AddRMSNorm(torch.autograd.Function):
    """(s, norm(s)) for s = residual + delta, residual fp32, delta fp16 (solution/rmsnorm.py:104-144)."""

    @staticmethod
    def forward(ctx, residual, delta, weight, eps, to_half):
        _check(residual, weight)
        if delta.dtype != torch.float16 or delta.shape != residual.shape:
            raise TypeError("hackaton_b200: add_rms_norm adds an fp16 tensor of the residual's shape")
        shape = residual.shape
        r2 = residual.reshape(-1, shape[-1]).contiguous()
        d2 = delta.reshape(-1, shape[-1]).contiguous()
        weight = weight.contiguous()
        out, rstd, total = _forward(r2, d2, weight, eps, to_half)
        ctx.save_for_backward(total, weight, rstd)
        ctx.shape, ctx.delta_dtype = shape, delta.dtype
        return total.reshape(shape), out.reshape(shape)

    @staticmethod
    def backward(ctx, d_total, dy):
        total, weight, rstd = ctx.saved_tensors
        dy2 = dy.reshape(total.shape).contiguous()
        d_total = d_total.reshape(total.shape).to(total.dtype).contiguous()
        dx = _backward(total, weight, rstd, dy2, d_total)
        dweight = _dweight(dy2, total, rstd, weight) if ctx.needs_input_grad[2] else None
        dx = dx.reshape(ctx.shape)
        return dx, dx.to(ctx.delta_dtype), dweight, None, None


def add_rms_norm(residual, delta, weight, eps, to_half=False):
    """(residual + delta, rms_norm(residual + delta)) in one pass (solution/rmsnorm.py:147-150)."""
    return AddRMSNorm.apply(residual, delta, weight, eps, to_half)
