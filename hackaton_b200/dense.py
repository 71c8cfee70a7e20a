"""Linear with a plain fp16 weight through the library's tcgen05 pipeline.

The one fp16 matrix product of the reference's step that is not an NF4 projection is the lm_head
(the tied embedding table, 151,936 x 1536 in Qwen2.5-1.5B), which the reference hands to cuBLAS
chunk by chunk (solution/lm_loss.py:31-40). Here it runs through the same kernel as the NF4
projections, with the weight tiles brought by TMA instead of decoded (csrc/gemm.cu, DENSE).
"""

from __future__ import annotations

import torch

from . import _lib
from .nf4 import _rows_view, _stream_ptr, _workspace


def fp16_linear(x, weight, transposed=False, bias=None, out=None):
    """transposed=False: y = x . weightᵀ (+ bias), weight [N, K], x [..., K] -> [..., N]
    transposed=True:  y = x . weight,          weight [N, K], x [..., N] -> [..., K]
    fp16 in, fp32 accumulate, fp16 out. `out`: an fp16 [rows, cols] tensor to fill (row stride a
    multiple of 8 elements)."""
    if x.dtype != torch.float16 or weight.dtype != torch.float16:
        raise TypeError(f"hackaton_b200: fp16_linear computes in fp16, got {x.dtype} and {weight.dtype}")
    if not (x.is_cuda and weight.is_cuda):
        raise ValueError("hackaton_b200: fp16_linear needs CUDA tensors (there is no CPU path)")
    if weight.dim() != 2:
        raise ValueError("hackaton_b200: fp16_linear takes a 2-D weight")
    if weight.stride(1) != 1 or weight.stride(0) % 8 != 0 or weight.data_ptr() % 16 != 0:
        weight = weight.contiguous()
    n, k = weight.shape
    in_cols, out_cols = (n, k) if transposed else (k, n)
    if x.shape[-1] != in_cols:
        raise ValueError(f"input has {x.shape[-1]} features, weight expects {in_cols}")
    x2 = _rows_view(x, in_cols)
    m = x2.shape[0]
    if out is None:
        y = torch.empty((m, out_cols), dtype=torch.float16, device=x.device)
    else:
        y = out
        if y.dtype != torch.float16 or tuple(y.shape) != (m, out_cols) or y.stride(1) != 1:
            raise ValueError("hackaton_b200: `out` must be an fp16 [rows, cols] tensor with unit column stride")
    if m == 0:
        return y if out is not None else y.reshape(*x.shape[:-1], out_cols)
    if bias is not None:
        bias = bias.to(torch.float16).contiguous()
    ws, ws_bytes = _workspace(x.device, n, k, m, bool(transposed))
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().nf4b200_fp16_linear(
            weight.data_ptr(), n, k, weight.stride(0), x2.data_ptr(), m, x2.stride(0),
            int(bool(transposed)), None if bias is None else bias.data_ptr(), y.data_ptr(),
            y.stride(0), ws, ws_bytes, _stream_ptr(x.device)))
    return y if out is not None else y.reshape(*x.shape[:-1], out_cols)
