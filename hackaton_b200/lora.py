"""LoRA (rank 16) on top of the fused NF4 linear.

    y = x . Wᵀ + bias + scaling * (x_l . Aᵀ) . Bᵀ          A: [16, K], B: [N, 16]

with x_l = dropout(x) in training (peft's `lora_dropout`), x_l = x otherwise. The reference runs
this as peft's stock `Linear.forward` around `bnb.nn.Linear4bit` (third-party code, configured at
README.md:91 and task/task.yaml:18-21: r=16, alpha=32, targets q_proj / v_proj): several small
cuBLAS launches plus scale and add per layer. Here the rank-16 update is one extra K=16 step of
the same tcgen05 GEMM that consumes the NF4 codes, in the forward and in the input gradient.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .nf4 import _rows_view, _stream_ptr, linear_backward_dx, linear_forward

RANK = 16


def lora_down(inp, p, p_is_rank_major, scaling):
    """fp16 [M, 16] = scaling * inp[M, C] . P, P given as lora_A [16, C] (rank-major) or
    lora_B [C, 16]."""
    c = inp.shape[-1]
    i2 = _rows_view(inp, c)
    p = p.detach()
    if p.dtype != torch.float16 or not p.is_contiguous():
        p = p.to(torch.float16).contiguous()
    if p_is_rank_major:
        assert tuple(p.shape) == (RANK, c), (p.shape, c)
        stride_r, stride_c = c, 1
    else:
        assert tuple(p.shape) == (c, RANK), (p.shape, c)
        stride_r, stride_c = 1, RANK
    out = torch.empty((i2.shape[0], RANK), dtype=torch.float16, device=inp.device)
    with torch.cuda.device(inp.device):
        _lib.check(_lib.lib().nf4b200_lora_down(i2.data_ptr(), i2.shape[0], c, i2.stride(0),
                                                p.data_ptr(), stride_r, stride_c, float(scaling),
                                                out.data_ptr(), _stream_ptr(inp.device)))
    return out


def lora_grad(z, s, rank_major_out):
    """fp32 weight gradient: zᵀ . s laid out [16, C] (rank_major_out) or [C, 16]."""
    c = z.shape[-1]
    z2 = _rows_view(z, c)
    shape = (RANK, c) if rank_major_out else (c, RANK)
    out = torch.zeros(shape, dtype=torch.float32, device=z.device)
    stride_r, stride_c = (c, 1) if rank_major_out else (1, RANK)
    with torch.cuda.device(z.device):
        _lib.check(_lib.lib().nf4b200_lora_grad(z2.data_ptr(), z2.shape[0], c, z2.stride(0),
                                                s.data_ptr(), out.data_ptr(), stride_r, stride_c,
                                                _stream_ptr(z.device)))
    return out


def _arr(ctype, values):
    return (ctype * len(values))(*values)


def lora_down_batch(inputs, ps, p_is_rank_major, scalings):
    """lora_down for several (input, P) pairs with the same number of rows in one launch
    (nf4b200_lora_down_batch). Returns the list of fp16 [M, 16] results."""
    n = len(inputs)
    if n == 1:
        return [lora_down(inputs[0], ps[0], p_is_rank_major, scalings[0])]
    i2s, p16s, cs = [], [], []
    for inp, p in zip(inputs, ps):
        c = inp.shape[-1]
        i2s.append(_rows_view(inp, c))
        p = p.detach()
        if p.dtype != torch.float16 or not p.is_contiguous():
            p = p.to(torch.float16).contiguous()
        assert tuple(p.shape) == ((RANK, c) if p_is_rank_major else (c, RANK)), (p.shape, c)
        p16s.append(p)
        cs.append(c)
    m = i2s[0].shape[0]
    assert all(t.shape[0] == m for t in i2s)
    device = inputs[0].device
    out = torch.empty((n, m, RANK), dtype=torch.float16, device=device)
    outs = [out[i] for i in range(n)]
    stride_r = [c if p_is_rank_major else 1 for c in cs]
    stride_c = [1 if p_is_rank_major else RANK for _ in cs]
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    with torch.cuda.device(device):
        _lib.check(_lib.lib().nf4b200_lora_down_batch(
            n, _arr(vp, [t.data_ptr() for t in i2s]), m, _arr(i64, cs),
            _arr(i64, [t.stride(0) for t in i2s]), _arr(vp, [t.data_ptr() for t in p16s]),
            _arr(i64, stride_r), _arr(i64, stride_c), _arr(ctypes.c_float, [float(v) for v in scalings]),
            _arr(vp, [t.data_ptr() for t in outs]), _stream_ptr(device)))
    return outs


def lora_grad_batch(zs, ss, rank_major_outs):
    """lora_grad for several (z, s) pairs in one launch (nf4b200_lora_grad_batch); one zeroed
    fp32 buffer holds all results. Returns the list of gradients, [16, C] or [C, 16] each."""
    n = len(zs)
    if n == 1:
        return [lora_grad(zs[0], ss[0], rank_major_outs[0])]
    z2s = [_rows_view(z, z.shape[-1]) for z in zs]
    cs = [z.shape[-1] for z in zs]
    device = zs[0].device
    sizes = [(c * RANK + 63) // 64 * 64 for c in cs]         # 256-byte aligned pieces
    flat = torch.zeros(sum(sizes), dtype=torch.float32, device=device)
    outs, at = [], 0
    for c, size, rm in zip(cs, sizes, rank_major_outs):
        outs.append(flat[at:at + c * RANK].view((RANK, c) if rm else (c, RANK)))
        at += size
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    with torch.cuda.device(device):
        _lib.check(_lib.lib().nf4b200_lora_grad_batch(
            n, _arr(vp, [t.data_ptr() for t in z2s]), _arr(i64, [t.shape[0] for t in z2s]),
            _arr(i64, cs), _arr(i64, [t.stride(0) for t in z2s]),
            _arr(vp, [t.data_ptr() for t in ss]), _arr(vp, [t.data_ptr() for t in outs]),
            _arr(i64, [c if rm else 1 for c, rm in zip(cs, rank_major_outs)]),
            _arr(i64, [1 if rm else RANK for rm in rank_major_outs]), _stream_ptr(device)))
    return outs


class NF4LoRALinear(torch.autograd.Function):
    """Frozen NF4 base weight + trainable rank-16 A, B. `x_lora` is the input of the LoRA branch:
    pass `x` itself when there is no dropout (then the input gradient is one fused GEMM)."""

    @staticmethod
    def forward(ctx, x, x_lora, packed, bias, state, lora_a, lora_b, scaling):
        same = x_lora is x or (x_lora.data_ptr() == x.data_ptr() and x_lora.shape == x.shape
                               and x_lora.stride() == x.stride())
        xa = lora_down(x_lora, lora_a, True, scaling)          # scaling * x_l . Aᵀ  [M,16]
        b16 = lora_b.detach().to(torch.float16).contiguous()
        y = linear_forward(x, packed, bias, state, xa=xa, lora_b=b16)
        ctx.packed, ctx.state, ctx.scaling, ctx.same = packed, state, float(scaling), same
        ctx.bias_dtype = None if bias is None else bias.dtype
        ctx.save_for_backward(x_lora, xa, lora_a, lora_b)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        x_lora, xa, lora_a, lora_b = ctx.saved_tensors
        need_x, need_xl = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_a, need_b = ctx.needs_input_grad[5], ctx.needs_input_grad[6]
        grad_x = grad_xl = grad_bias = grad_a = grad_b = None
        u = None
        if need_x or need_xl or need_a:
            u = lora_down(grad_output, lora_b, False, ctx.scaling)   # scaling * dy . B  [M,16]
        a16 = lora_a.detach().to(torch.float16).contiguous()
        if ctx.same:
            if need_x or need_xl:
                grad_x = linear_backward_dx(grad_output, ctx.packed, ctx.state, u=u, lora_a=a16)
        else:
            if need_x:
                grad_x = linear_backward_dx(grad_output, ctx.packed, ctx.state)
            if need_xl:  # the dropout branch keeps its own gradient: u . A
                grad_xl = (u.reshape(-1, RANK) @ a16).reshape(x_lora.shape)
        if need_a:
            grad_a = lora_grad(x_lora, u, True).to(lora_a.dtype)
        if need_b:
            grad_b = lora_grad(grad_output, xa, False).to(lora_b.dtype)
        if ctx.needs_input_grad[3]:
            grad_bias = grad_output.reshape(-1, grad_output.shape[-1]).sum(0, dtype=ctx.bias_dtype)
        return grad_x, grad_xl, None, grad_bias, None, grad_a, grad_b, None


def nf4_lora_linear(x, packed, bias, state, lora_a, lora_b, scaling, x_lora=None):
    """y = x . Wᵀ + bias + scaling * (x_lora . Aᵀ) . Bᵀ; x_lora defaults to x."""
    if x_lora is None:
        x_lora = x
    return NF4LoRALinear.apply(x, x_lora, packed.reshape(-1), bias, state, lora_a, lora_b, scaling)
