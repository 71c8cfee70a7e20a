"""Cross-entropy straight from the lm_head's logits, and lm_head + loss in chunks of rows.

Mirrors the reference's `ce_stats` / `ce_grad` / `fused_cross_entropy` (solution/kernels.py:173-238)
and `linear_cross_entropy` (solution/lm_loss.py:27-62): the statistics pass and the gradient pass
are this library's kernels; the two matmuls of a chunk are plain fp16 GEMMs on an unquantised
weight (the tied embedding table), i.e. library calls, as in the reference.
"""

from __future__ import annotations

import torch

from . import _lib
from .nf4 import _stream_ptr

CHUNK_ROWS = 256      # solution/lm_loss.py:27
GRAD_SCALE = 1024.0   # solution/lm_loss.py:28


def _dtype_code(logits):
    if not logits.is_cuda:
        raise ValueError("hackaton_b200: the cross-entropy kernels need CUDA tensors (there is no CPU path)")
    if logits.dtype == torch.float16:
        return _lib.F16
    if logits.dtype == torch.float32:
        return _lib.F32
    raise TypeError(f"hackaton_b200: logits must be fp16 or fp32, got {logits.dtype}")


def ce_grad(logits, targets, lse, scale, grad):
    """grad = scale * (softmax(logits) - onehot(targets)) per row, 0 for rows with target < 0;
    `grad` may be `logits` itself (solution/kernels.py:173-179)."""
    rows, vocab = logits.shape
    with torch.cuda.device(logits.device):
        _lib.check(_lib.lib().nf4b200_ce_grad(
            logits.data_ptr(), _dtype_code(logits), targets.data_ptr(), lse.data_ptr(), scale.data_ptr(),
            grad.data_ptr(), rows, vocab, _stream_ptr(logits.device)))


def ce_stats(logits, targets, want_entropy, out=None):
    """Per-row logsumexp, loss (0 for rows with target < 0) and, if asked, entropy of (rows,
    vocab) logits. `out` = (lse, loss, entropy, argmax) buffers to fill, argmax included
    (solution/kernels.py:182-204)."""
    rows, vocab = logits.shape
    if targets.dtype != torch.int64:
        raise TypeError("hackaton_b200: targets must be int64")
    if out is not None:
        lse, loss, entropy, argmax = out
    else:
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        loss = torch.empty_like(lse)
        entropy = torch.empty_like(lse) if want_entropy else None
        argmax = None
    with torch.cuda.device(logits.device):
        _lib.check(_lib.lib().nf4b200_ce_stats(
            logits.data_ptr(), _dtype_code(logits), targets.data_ptr(), lse.data_ptr(), loss.data_ptr(),
            None if entropy is None else entropy.data_ptr(),
            None if argmax is None else argmax.data_ptr(), rows, vocab, _stream_ptr(logits.device)))
    return lse, loss, entropy


class FusedCrossEntropy(torch.autograd.Function):
    """sum over rows of (logsumexp - logit[target]) / denom, rows with target < 0 ignored
    (solution/kernels.py:207-231)."""

    @staticmethod
    def forward(ctx, logits, targets, denom, inplace_grad):
        lse, losses, _ = ce_stats(logits, targets, False)
        ctx.save_for_backward(logits, targets, lse, denom)
        ctx.inplace_grad = inplace_grad
        return losses.sum() / denom

    @staticmethod
    def backward(ctx, grad_output):
        logits, targets, lse, denom = ctx.saved_tensors
        scale = (grad_output / denom).to(torch.float32).reshape(1)
        grad = logits if ctx.inplace_grad else torch.empty_like(logits)
        ce_grad(logits, targets, lse, scale, grad)
        return grad, None, None, None


def fused_cross_entropy(logits, targets, denom, inplace_grad=False):
    """solution/kernels.py:234-238."""
    return FusedCrossEntropy.apply(logits.contiguous(), targets, denom, inplace_grad)


def _chunks(hidden, weight, targets, lse, losses, entropy, argmax, unit, grad_hidden):
    rows = hidden.shape[0]
    for start in range(0, rows, CHUNK_ROWS):
        part = slice(start, min(start + CHUNK_ROWS, rows))
        logits = torch.nn.functional.linear(hidden[part], weight)
        ce_stats(logits, targets[part], True, out=(lse[part], losses[part], entropy[part], argmax[part]))
        ce_grad(logits, targets[part], lse[part], unit, logits)   # 1024 (p - onehot), in place
        torch.mm(logits, weight, out=grad_hidden[part])


class LinearCrossEntropy(torch.autograd.Function):
    """lm_head and the loss without the (tokens, vocab) logits (solution/lm_loss.py:45-62): the
    gradient with respect to `hidden` is formed in the forward, chunk by chunk, and scaled in the
    backward; the weight is frozen."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, denom):
        rows, device = hidden.shape[0], hidden.device
        lse = torch.empty(rows, dtype=torch.float32, device=device)
        losses, entropy = torch.empty_like(lse), torch.empty_like(lse)
        argmax = torch.empty(rows, dtype=torch.int64, device=device)
        unit = torch.full((1,), GRAD_SCALE, dtype=torch.float32, device=device)
        grad_hidden = torch.empty_like(hidden)
        with torch.autocast("cuda", enabled=False):
            _chunks(hidden, weight, targets, lse, losses, entropy, argmax, unit, grad_hidden)
        ctx.save_for_backward(grad_hidden, denom)
        ctx.mark_non_differentiable(losses, entropy, argmax)
        return losses.sum() / denom, losses, entropy, argmax

    @staticmethod
    def backward(ctx, grad_output, _losses, _entropy, _argmax):
        grad_hidden, denom = ctx.saved_tensors
        scale = (grad_output.float() / (denom * GRAD_SCALE)).reshape(1, 1)
        return (grad_hidden.float() * scale).to(grad_hidden.dtype), None, None, None


def linear_cross_entropy(hidden, weight, targets, denom):
    """(loss, per-row losses, entropy, argmax) of hidden @ weight^T against `targets`
    (solution/lm_loss.py:65-67)."""
    return LinearCrossEntropy.apply(hidden.contiguous(), weight, targets, denom)
