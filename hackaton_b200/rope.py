"""Rotary embedding + grouped-query expansion of the packed q / k / v projections: the step
right after the q/k/v GEMM.

Mirrors the reference's `qkv_rotate` / `QKVRotate` (solution/attention.py:149-192): one kernel
launch forward, one backward, outputs fp16 with every k / v head repeated heads / kv_heads times,
packed (N, H, D) or padded (B, H, T, D).
"""

from __future__ import annotations

import torch

from . import _lib
from .nf4 import _stream_ptr


def _launch(q, k, v, qo, ko, vo, cos, sin, scb, b_idx, t_idx, tokens, seq, heads, kv_heads, dim,
            padded, backward, proj_dtype):
    with torch.cuda.device(qo.device):
        _lib.check(_lib.lib().nf4b200_qkv_rotate(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), qo.data_ptr(), ko.data_ptr(), vo.data_ptr(),
            cos.data_ptr(), sin.data_ptr(), scb, cos.stride(1), b_idx.data_ptr(), t_idx.data_ptr(),
            tokens, seq, heads, kv_heads, dim, int(padded), int(backward),
            _lib.F32 if proj_dtype == torch.float32 else _lib.F16, _stream_ptr(qo.device)))


class QKVRotate(torch.autograd.Function):
    """Packed (q, k, v) projections (N, heads * D) -> rotated, fp16, GQA-expanded heads."""

    @staticmethod
    def forward(ctx, q, k, v, cos, sin, b_idx, t_idx, batch, seq, heads, kv_heads, padded):
        if not q.is_cuda:
            raise ValueError("hackaton_b200: qkv_rotate needs CUDA tensors (there is no CPU path)")
        if q.dtype not in (torch.float16, torch.float32) or k.dtype != q.dtype or v.dtype != q.dtype:
            raise TypeError(f"hackaton_b200: qkv_rotate takes fp16 or fp32 projections, got {q.dtype}")
        if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.dim() != 3:
            raise TypeError("hackaton_b200: qkv_rotate takes fp32 cos / sin of shape (1 or B, T, D)")
        dim = q.shape[-1] // heads
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        cos, sin = cos.contiguous(), sin.contiguous()
        b_idx, t_idx = b_idx.to(torch.int32).contiguous(), t_idx.to(torch.int32).contiguous()
        scb = 0 if cos.shape[0] == 1 else cos.stride(0)
        tokens = q.shape[0]
        if padded:
            qo = torch.zeros(batch, heads, seq, dim, dtype=torch.float16, device=q.device)
            ko, vo = torch.zeros_like(qo), torch.zeros_like(qo)
        else:
            qo = torch.empty(tokens, heads, dim, dtype=torch.float16, device=q.device)
            ko, vo = torch.empty_like(qo), torch.empty_like(qo)
        _launch(q, k, v, qo, ko, vo, cos, sin, scb, b_idx, t_idx, tokens, seq, heads, kv_heads, dim,
                padded, False, q.dtype)
        ctx.save_for_backward(cos, sin, b_idx, t_idx)
        ctx.meta = (seq, scb, heads, kv_heads, dim, q.dtype, bool(padded))
        return qo, ko, vo

    @staticmethod
    def backward(ctx, dq, dk, dv):
        cos, sin, b_idx, t_idx = ctx.saved_tensors
        seq, scb, heads, kv_heads, dim, dtype, padded = ctx.meta
        tokens = b_idx.shape[0]
        dq, dk, dv = (g.to(torch.float16).contiguous() for g in (dq, dk, dv))
        dq_in = torch.empty(tokens, heads * dim, dtype=dtype, device=dq.device)
        dk_in = torch.empty(tokens, kv_heads * dim, dtype=dtype, device=dq.device)
        dv_in = torch.empty_like(dk_in)
        _launch(dq, dk, dv, dq_in, dk_in, dv_in, cos, sin, scb, b_idx, t_idx, tokens, seq, heads,
                kv_heads, dim, padded, True, dtype)
        return (dq_in, dk_in, dv_in) + (None,) * 9


def qkv_rotate(q, k, v, cos, sin, b_idx, t_idx, batch, seq, heads, kv_heads, padded=False):
    """solution/attention.py:191-192."""
    return QKVRotate.apply(q, k, v, cos, sin, b_idx, t_idx, batch, seq, heads, kv_heads, padded)
