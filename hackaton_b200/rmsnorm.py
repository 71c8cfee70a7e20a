"""RMSNorm and add + RMSNorm on the fp32 residual stream: the step right before the q/k/v and
gate/up projections, which hands them their fp16 input.

Same surface as the reference's `rms_norm` / `add_rms_norm` (solution/rmsnorm.py:52-150; used by
solution/packed.py:88-115) without the host-offload option: one kernel pass per direction, and
besides the normalised tensor only one fp32 number per row is kept for the gradient pass.
"""

from __future__ import annotations

import torch

from . import _lib
from ._autograd import call
from .nf4 import _stream_ptr


def _out_code(dtype):
    return _lib.F16 if dtype == torch.float16 else _lib.F32


def launch_forward(x2, delta2, weight, eps, to_half):
    """One forward pass over rows of fp32 `x2` (+ fp16 `delta2`). Returns (normalised rows in fp16
    or fp32, 1/rms per row, the fp32 sum x2 + delta2 or None)."""
    rows, hidden = x2.shape
    device = x2.device
    out = torch.empty((rows, hidden), dtype=torch.float16 if to_half else torch.float32, device=device)
    rstd = torch.empty(rows, dtype=torch.float32, device=device)
    total = None if delta2 is None else torch.empty_like(x2)
    with torch.cuda.device(device):
        _lib.check(_lib.lib().nf4b200_rmsnorm_fwd(
            x2.data_ptr(), None if delta2 is None else delta2.data_ptr(), weight.data_ptr(),
            None if total is None else total.data_ptr(), out.data_ptr(), _out_code(out.dtype),
            rstd.data_ptr(), rows, hidden, float(eps), _stream_ptr(device)))
    return out, rstd, total


def launch_backward(x2, weight, rstd, dy2, d_total=None):
    """Gradient with respect to the normalised rows' input; `d_total` (fp32, optional) is added in
    the same pass (the gradient that reached the sum directly)."""
    rows, hidden = x2.shape
    dx = torch.empty_like(x2)
    with torch.cuda.device(x2.device):
        _lib.check(_lib.lib().nf4b200_rmsnorm_bwd(
            x2.data_ptr(), weight.data_ptr(), rstd.data_ptr(), dy2.data_ptr(), _out_code(dy2.dtype),
            None if d_total is None else d_total.data_ptr(), dx.data_ptr(), rows, hidden,
            _stream_ptr(x2.device)))
    return dx


def _rows(t):
    return t.reshape(-1, t.shape[-1]).contiguous()


def _validate(x, weight):
    if not (x.is_cuda and weight.is_cuda):
        raise ValueError("hackaton_b200: RMSNorm needs CUDA tensors (there is no CPU path)")
    if x.dtype != torch.float32 or weight.dtype != torch.float32:
        raise TypeError(f"hackaton_b200: RMSNorm runs on the fp32 stream, got {x.dtype}, {weight.dtype}")
    if weight.numel() != x.shape[-1]:
        raise ValueError("hackaton_b200: RMSNorm weight does not match the last dimension")


class _NormOp:
    """weight * x / rms(x), optionally of x = residual + delta with the sum as a second output.
    The frozen norm weight's gradient (not on the fine-tuning path) is a plain torch reduction,
    as in the reference (solution/rmsnorm.py:93-95)."""

    def __init__(self, eps, to_half, with_delta):
        self.eps, self.to_half, self.with_delta = eps, to_half, with_delta

    def run(self, keep, x, weight, delta=None):
        _validate(x, weight)
        if self.with_delta and (delta.dtype != torch.float16 or delta.shape != x.shape):
            raise TypeError("hackaton_b200: add_rms_norm adds an fp16 tensor of the residual's shape")
        weight = weight.contiguous()
        out, rstd, total = launch_forward(_rows(x), _rows(delta) if self.with_delta else None,
                                          weight, self.eps, self.to_half)
        normed_input = total if self.with_delta else _rows(x)
        keep(normed_input, weight, rstd, shape=x.shape)
        if self.with_delta:
            return total.reshape(x.shape), out.reshape(x.shape)
        return out.reshape(x.shape)

    def grad(self, kept, *grads):
        rows, weight, rstd = kept.tensors
        if self.with_delta:
            d_total, dy = grads
            d_total = d_total.reshape(rows.shape).to(torch.float32).contiguous()
        else:
            (dy,), d_total = grads, None
        dy2 = dy.reshape(rows.shape).contiguous()
        dx = launch_backward(rows, weight, rstd, dy2, d_total).reshape(kept.shape)
        dweight = None
        if kept.wants[1]:
            dweight = (dy2.float() * (rows * rstd[:, None])).sum(dim=0).to(weight.dtype)
        if self.with_delta:
            return dx, dweight, dx.to(torch.float16)
        return dx, dweight


def rms_norm(x, weight, eps, to_half=False):
    """weight * (x * rsqrt(mean(x^2) + eps)) for fp32 x; fp16 output with `to_half`
    (solution/rmsnorm.py:52-101)."""
    return call(_NormOp(eps, to_half, False), x, weight)


def add_rms_norm(residual, delta, weight, eps, to_half=False):
    """(residual + delta, rms_norm(residual + delta)) in one pass; residual fp32, delta fp16
    (solution/rmsnorm.py:104-150)."""
    return call(_NormOp(eps, to_half, True), residual, weight, delta)
