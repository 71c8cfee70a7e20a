"""Cross-entropy straight from the lm_head's logits, and lm_head + loss over row chunks.

Same surface as the reference's `ce_stats` / `ce_grad` / `fused_cross_entropy`
(solution/kernels.py:173-238) and `linear_cross_entropy` (solution/lm_loss.py:27-67). The
statistics pass and the gradient pass are this library's kernels (csrc/cross_entropy.cu), and so
are the two fp16 matrix products of a chunk (`dense.fp16_linear`: the tcgen05 kernel of the NF4
projections with the weight tiles brought by TMA).
"""

from __future__ import annotations

import torch

from . import _lib
from ._autograd import call
from .dense import fp16_linear
from .nf4 import _stream_ptr

CHUNK_ROWS = 256      # rows of logits alive at a time (solution/lm_loss.py:27)
GRAD_SCALE = 1024.0   # the chunk gradients are kept in fp16 at this scale (solution/lm_loss.py:28)


def _dtype_code(logits):
    if not logits.is_cuda:
        raise ValueError("hackaton_b200: the cross-entropy kernels need CUDA tensors (there is no CPU path)")
    if logits.dtype == torch.float16:
        return _lib.F16
    if logits.dtype == torch.float32:
        return _lib.F32
    raise TypeError(f"hackaton_b200: logits must be fp16 or fp32, got {logits.dtype}")


def _opt_ptr(t):
    return None if t is None else t.data_ptr()


def ce_stats(logits, targets, want_entropy, out=None):
    """Per-row logsumexp, loss (0 for rows with target < 0) and, if asked, entropy of (rows,
    vocab) logits. `out` = (lse, loss, entropy, argmax) buffers to fill instead of new ones;
    the argmax is only written there (solution/kernels.py:182-204)."""
    rows, vocab = logits.shape
    if targets.dtype != torch.int64:
        raise TypeError("hackaton_b200: targets must be int64")
    if out is None:
        fresh = lambda: torch.empty(rows, dtype=torch.float32, device=logits.device)  # noqa: E731
        out = (fresh(), fresh(), fresh() if want_entropy else None, None)
    lse, loss, entropy, argmax = out
    with torch.cuda.device(logits.device):
        _lib.check(_lib.lib().nf4b200_ce_stats(
            logits.data_ptr(), _dtype_code(logits), targets.data_ptr(), lse.data_ptr(),
            loss.data_ptr(), _opt_ptr(entropy), _opt_ptr(argmax), rows, vocab,
            _stream_ptr(logits.device)))
    return lse, loss, entropy


def ce_grad(logits, targets, lse, scale, grad):
    """grad = scale * (softmax(logits) - onehot(targets)) per row, 0 for rows with target < 0;
    `scale` is one fp32 number on the device; `grad` may be `logits` itself
    (solution/kernels.py:173-179)."""
    rows, vocab = logits.shape
    with torch.cuda.device(logits.device):
        _lib.check(_lib.lib().nf4b200_ce_grad(
            logits.data_ptr(), _dtype_code(logits), targets.data_ptr(), lse.data_ptr(),
            scale.data_ptr(), grad.data_ptr(), rows, vocab, _stream_ptr(logits.device)))


class _LossFromLogits:
    """sum over rows of (logsumexp - logit[target]) / denom; the gradient may overwrite the
    logits."""

    def __init__(self, overwrite_logits):
        self.overwrite_logits = overwrite_logits

    def run(self, keep, logits, targets, denom):
        lse, per_row, _ = ce_stats(logits, targets, False)
        keep(logits, targets, lse, denom)
        return per_row.sum() / denom

    def grad(self, kept, upstream):
        logits, targets, lse, denom = kept.tensors
        d_logits = logits if self.overwrite_logits else torch.empty_like(logits)
        ce_grad(logits, targets, lse, (upstream / denom).float().reshape(1), d_logits)
        return d_logits, None, None


def fused_cross_entropy(logits, targets, denom, inplace_grad=False):
    """Mean-style loss of (rows, vocab) logits, rows with target < 0 ignored
    (solution/kernels.py:207-238)."""
    return call(_LossFromLogits(bool(inplace_grad)), logits.contiguous(), targets, denom)


def _head_products(hidden_rows, weight):
    """The two matrix products of one chunk: logits = hidden_rows . weightᵀ, and, once the logits
    have been turned into their gradient, d_hidden = d_logits . weight. fp16 weights (the model's
    own lm_head) go through this library's tcgen05 kernel; other dtypes (a test in fp32) use
    torch's matmul."""
    if hidden_rows.dtype == torch.float16 and weight.dtype == torch.float16:
        return (fp16_linear(hidden_rows, weight),
                lambda d_logits, out: fp16_linear(d_logits, weight, transposed=True, out=out))
    return (torch.nn.functional.linear(hidden_rows, weight),
            lambda d_logits, out: torch.mm(d_logits, weight, out=out))


class _HeadAndLoss:
    """lm_head + loss without ever holding the (tokens, vocab) logits: walks the rows in chunks;
    per chunk the logits are made, reduced to their statistics, turned in place into
    GRAD_SCALE * (softmax - onehot) and multiplied back through the (frozen) head weight, so the
    gradient with respect to `hidden` exists when the forward ends and the backward only rescales
    it (solution/lm_loss.py:31-62)."""

    def run(self, keep, hidden, weight, targets, denom):
        rows, device = hidden.shape[0], hidden.device
        stats = {name: torch.empty(rows, dtype=torch.float32, device=device)
                 for name in ("lse", "loss", "entropy")}
        argmax = torch.empty(rows, dtype=torch.int64, device=device)
        d_hidden = torch.empty_like(hidden)
        unit = torch.full((1,), GRAD_SCALE, dtype=torch.float32, device=device)
        with torch.autocast("cuda", enabled=False):
            for lo in range(0, rows, CHUNK_ROWS):
                rs = slice(lo, min(lo + CHUNK_ROWS, rows))
                logits, back = _head_products(hidden[rs], weight)
                ce_stats(logits, targets[rs], True,
                         out=(stats["lse"][rs], stats["loss"][rs], stats["entropy"][rs], argmax[rs]))
                ce_grad(logits, targets[rs], stats["lse"][rs], unit, logits)
                back(logits, d_hidden[rs])
        keep(d_hidden, denom)
        keep.constant(stats["loss"], stats["entropy"], argmax)
        return stats["loss"].sum() / denom, stats["loss"], stats["entropy"], argmax

    def grad(self, kept, upstream, *_unused):
        d_hidden, denom = kept.tensors
        factor = (upstream.float() / (denom * GRAD_SCALE)).reshape(1, 1)
        return (d_hidden.float() * factor).to(d_hidden.dtype), None, None, None


def linear_cross_entropy(hidden, weight, targets, denom):
    """(loss, per-row losses, entropy, argmax) of hidden @ weightᵀ against `targets`
    (solution/lm_loss.py:65-67)."""
    return call(_HeadAndLoss(), hidden.contiguous(), weight, targets, denom)
