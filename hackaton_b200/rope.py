"""Rotary embedding + grouped-query expansion of the packed q / k / v projections: the step
right after the q/k/v GEMM.

Same surface as the reference's `qkv_rotate` (solution/attention.py:149-192): one kernel launch
forward, one backward, outputs fp16 with every k / v head repeated heads / kv_heads times, packed
(N, H, D) or padded (B, H, T, D).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._autograd import call
from .nf4 import _stream_ptr


@dataclass
class RotateGeometry:
    """Everything about one rotation that is not a tensor."""
    tokens: int
    seq: int
    heads: int
    kv_heads: int
    dim: int
    padded: bool
    batch_stride: int          # elements between the cos / sin tables of two batches, 0 if shared
    proj_dtype: torch.dtype    # type of the projections (forward input, backward output)


def launch(src, dst, cos, sin, b_idx, t_idx, geo: RotateGeometry, backward: bool):
    """src, dst: (q, k, v) triples. Forward reads the projections and writes the expanded fp16
    heads; backward reads the heads' gradients and writes the projections' gradients."""
    device = dst[0].device
    with torch.cuda.device(device):
        _lib.check(_lib.lib().nf4b200_qkv_rotate(
            src[0].data_ptr(), src[1].data_ptr(), src[2].data_ptr(),
            dst[0].data_ptr(), dst[1].data_ptr(), dst[2].data_ptr(),
            cos.data_ptr(), sin.data_ptr(), geo.batch_stride, cos.stride(1),
            b_idx.data_ptr(), t_idx.data_ptr(), geo.tokens, geo.seq, geo.heads, geo.kv_heads,
            geo.dim, int(geo.padded), int(backward),
            _lib.F32 if geo.proj_dtype == torch.float32 else _lib.F16, _stream_ptr(device)))


class _RotateOp:
    def __init__(self, batch, seq, heads, kv_heads, padded):
        self.batch, self.seq, self.heads, self.kv_heads = batch, seq, heads, kv_heads
        self.padded = bool(padded)

    def run(self, keep, q, k, v, cos, sin, b_idx, t_idx):
        if not q.is_cuda:
            raise ValueError("hackaton_b200: qkv_rotate needs CUDA tensors (there is no CPU path)")
        if q.dtype not in (torch.float16, torch.float32) or k.dtype != q.dtype or v.dtype != q.dtype:
            raise TypeError(f"hackaton_b200: qkv_rotate takes fp16 or fp32 projections, got {q.dtype}")
        if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.dim() != 3:
            raise TypeError("hackaton_b200: qkv_rotate takes fp32 cos / sin of shape (1 or B, T, D)")
        cos, sin = cos.contiguous(), sin.contiguous()
        geo = RotateGeometry(tokens=q.shape[0], seq=self.seq, heads=self.heads, kv_heads=self.kv_heads,
                             dim=q.shape[-1] // self.heads, padded=self.padded,
                             batch_stride=0 if cos.shape[0] == 1 else cos.stride(0),
                             proj_dtype=q.dtype)
        index = tuple(t.to(torch.int32).contiguous() for t in (b_idx, t_idx))
        if self.padded:   # positions no token maps to stay zero
            shape, make = (self.batch, self.heads, self.seq, geo.dim), torch.zeros
        else:
            shape, make = (geo.tokens, self.heads, geo.dim), torch.empty
        heads_out = tuple(make(shape, dtype=torch.float16, device=q.device) for _ in range(3))
        launch(tuple(t.contiguous() for t in (q, k, v)), heads_out, cos, sin, *index, geo, False)
        keep(cos, sin, *index, geo=geo)
        return heads_out

    def grad(self, kept, *head_grads):
        cos, sin, b_idx, t_idx = kept.tensors
        geo = kept.geo
        src = tuple(g.to(torch.float16).contiguous() for g in head_grads)
        widths = (geo.heads, geo.kv_heads, geo.kv_heads)
        dst = tuple(torch.empty(geo.tokens, w * geo.dim, dtype=geo.proj_dtype, device=src[0].device)
                    for w in widths)
        launch(src, dst, cos, sin, b_idx, t_idx, geo, True)
        return dst + (None, None, None, None)


def qkv_rotate(q, k, v, cos, sin, b_idx, t_idx, batch, seq, heads, kv_heads, padded=False):
    """Packed (q, k, v) projections (N, heads * D) -> rotated, fp16, GQA-expanded heads
    (solution/attention.py:149-192)."""
    return call(_RotateOp(batch, seq, heads, kv_heads, padded), q, k, v, cos, sin, b_idx, t_idx)
