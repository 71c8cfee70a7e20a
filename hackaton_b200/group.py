"""Grouped launches for projections that sit side by side in the model.

In Qwen2 the q/k/v projections share the post-norm hidden state and gate/up share the MLP input
(the call sites the reference patches: solution/patches.py:32-41 and :98-99). Run one by one,
the small ones (k, v: 256 x 1536) leave most of a B200 idle. Here up to four NF4 weights with the
same number of input features go through ONE fused kernel launch:

    forward :  y_i = x . W_iᵀ (+ bias_i) (+ LoRA_i)        one x, one output per weight
    backward:  dx  = Σ_i dy_i . W_i (+ LoRA_i share)       one dx for the whole group

which is exactly what autograd computes for such a fan-out, only with fewer and fuller launches.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from .lora import RANK, lora_down_batch, lora_grad_batch
from .nf4 import _require, _rows_view, _stream_ptr, _ws_buffers, weight_ref

MAX_GROUP = 4


@dataclass
class Projection:
    """One member of a group: an NF4 weight and, optionally, its bias and LoRA pair."""
    packed: torch.Tensor
    state: object
    bias: Optional[torch.Tensor] = None
    lora_a: Optional[torch.Tensor] = None   # [16, K]
    lora_b: Optional[torch.Tensor] = None   # [N, 16]
    scaling: float = 1.0


_ws_need = {}


def _workspace(device, rows, cols, m, backward):
    key = (device.index, tuple(rows), cols, m, backward)
    need = _ws_need.get(key)
    if need is None:
        arr = (ctypes.c_int64 * len(rows))(*rows)
        with torch.cuda.device(device):
            need = int(_lib.lib().nf4b200_workspace_bytes_group(len(rows), arr, cols, m, int(backward)))
        if need < 0:
            _lib.check(need)
        _ws_need[key] = need
    if need == 0:
        return None, 0
    skey = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _ws_buffers.get(skey)
    if buf is None or buf.numel() < need:
        buf = torch.empty(max(need, 1 << 22), dtype=torch.uint8, device=device)
        _ws_buffers[skey] = buf
    return buf.data_ptr(), buf.numel()


def _refs(items):
    refs = []
    for packed, state in items:
        packed = packed.reshape(-1)
        _require(packed, state)
        refs.append(weight_ref(packed, state).prepare())
    cols = refs[0].cols
    if any(r.cols != cols for r in refs):
        raise ValueError("grouped projections must have the same number of input features")
    if not 1 <= len(refs) <= MAX_GROUP:
        raise ValueError(f"a group holds 1..{MAX_GROUP} projections, got {len(refs)}")
    return refs


def _ptr_array(values):
    return (ctypes.c_void_p * len(values))(*[None if v is None else v.data_ptr() for v in values])


def linear_forward_group(x, weights: Sequence, biases=None, xas=None, lora_bs=None):
    """weights: [(packed, state), ...]. Returns the list of outputs y_i = x . W_iᵀ (+ ...)."""
    refs = _refs(weights)
    n = len(refs)
    if x.dtype != torch.float16:
        raise TypeError(f"hackaton_b200: the fused NF4 linear computes in fp16, got {x.dtype}")
    cols = refs[0].cols
    x2 = _rows_view(x, cols)
    m = x2.shape[0]
    ys = [torch.empty((m, r.rows), dtype=torch.float16, device=x.device) for r in refs]
    if m == 0:
        return [y.reshape(*x.shape[:-1], y.shape[1]) for y in ys]
    biases = [None] * n if biases is None else [None if b is None else b.to(torch.float16).contiguous()
                                                 for b in biases]
    xas = [None] * n if xas is None else list(xas)
    lora_bs = [None] * n if lora_bs is None else list(lora_bs)
    ws, ws_bytes = _workspace(x.device, [r.rows for r in refs], cols, m, False)
    w_arr = (ctypes.POINTER(_lib.Weight) * n)(*[ctypes.pointer(r.struct) for r in refs])
    ldy = (ctypes.c_int64 * n)(*[y.stride(0) for y in ys])
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().nf4b200_linear_fwd_group(
            n, w_arr, x2.data_ptr(), m, x2.stride(0), _ptr_array(biases), _ptr_array(xas),
            _ptr_array(lora_bs), _ptr_array(ys), ldy, ws, ws_bytes, _stream_ptr(x.device)))
    return [y.reshape(*x.shape[:-1], y.shape[1]) for y in ys]


def linear_backward_dx_group(grads: Sequence[torch.Tensor], weights: Sequence, us=None, lora_as=None):
    """dx = Σ_i grads[i] . W_i (+ u_i . lora_a_i). grads[i]: fp16 [..., N_i]."""
    refs = _refs(weights)
    n = len(refs)
    g2 = []
    for g, r in zip(grads, refs):
        if g.dtype != torch.float16:
            raise TypeError(f"hackaton_b200: the fused NF4 linear computes in fp16, got {g.dtype}")
        g2.append(_rows_view(g, r.rows))
    m = g2[0].shape[0]
    cols = refs[0].cols
    dx = torch.empty((m, cols), dtype=torch.float16, device=g2[0].device)
    lead = grads[0].shape[:-1]
    if m == 0:
        return dx.reshape(*lead, cols)
    us = [None] * n if us is None else list(us)
    lora_as = [None] * n if lora_as is None else list(lora_as)
    device = g2[0].device
    ws, ws_bytes = _workspace(device, [r.rows for r in refs], cols, m, True)
    w_arr = (ctypes.POINTER(_lib.Weight) * n)(*[ctypes.pointer(r.struct) for r in refs])
    ldg = (ctypes.c_int64 * n)(*[g.stride(0) for g in g2])
    with torch.cuda.device(device):
        _lib.check(_lib.lib().nf4b200_linear_bwd_dx_group(
            n, w_arr, _ptr_array(g2), m, ldg, _ptr_array(us), _ptr_array(lora_as), dx.data_ptr(),
            dx.stride(0), ws, ws_bytes, _stream_ptr(device)))
    return dx.reshape(*lead, cols)


class NF4LinearGroup(torch.autograd.Function):
    """Autograd wrapper: inputs (x, projections, bias_0, A_0, B_0, bias_1, ...), one output per
    projection. Weights are frozen; gradients flow to x, the biases and the LoRA pairs."""

    @staticmethod
    def forward(ctx, x, projs, *params):
        n = len(projs)
        biases, las, lbs = params[0::3], params[1::3], params[2::3]
        xas, b16 = [None] * n, [None] * n
        with_lora = [i for i, a in enumerate(las) if a is not None]
        if with_lora:  # every adapter's scaling * x . Aᵀ in one launch
            downs = lora_down_batch([x] * len(with_lora), [las[i] for i in with_lora], True,
                                    [projs[i].scaling for i in with_lora])
            for i, xa in zip(with_lora, downs):
                xas[i] = xa
                b16[i] = lbs[i].detach().to(torch.float16).contiguous()
        ys = linear_forward_group(x, [(pr.packed, pr.state) for pr in projs], biases, xas, b16)
        ctx.projs, ctx.n = projs, n
        ctx.bias_dtypes = [None if b is None else b.dtype for b in biases]
        ctx.has_lora = [a is not None for a in las]
        saved = [x]
        for a, b, xa in zip(las, lbs, xas):
            if a is not None:
                saved += [a, b, xa]
        ctx.save_for_backward(*saved)
        return tuple(ys)

    @staticmethod
    def backward(ctx, *grads):
        saved = list(ctx.saved_tensors)
        x = saved.pop(0)
        projs = ctx.projs
        lora = []
        for has in ctx.has_lora:
            lora.append((saved.pop(0), saved.pop(0), saved.pop(0)) if has else None)
        grads = [g if g is not None else
                 torch.zeros(*x.shape[:-1], pr.state.shape[0], dtype=torch.float16, device=x.device)
                 for g, pr in zip(grads, projs)]
        us, a16 = [None] * len(projs), [None] * len(projs)
        with_lora = [i for i, lo in enumerate(lora) if lo is not None]
        if with_lora:  # every adapter's scaling * dy . B in one launch
            downs = lora_down_batch([grads[i] for i in with_lora], [lora[i][1] for i in with_lora],
                                    False, [projs[i].scaling for i in with_lora])
            for i, u in zip(with_lora, downs):
                us[i] = u
                a16[i] = lora[i][0].detach().to(torch.float16).contiguous()
        grad_x = None
        if ctx.needs_input_grad[0]:
            grad_x = linear_backward_dx_group(grads, [(pr.packed, pr.state) for pr in projs], us, a16)
        # all LoRA weight gradients of the group in one launch
        jobs = []  # (projection, "a" | "b", z, s, rank-major output)
        for i in with_lora:
            if ctx.needs_input_grad[3 + 3 * i]:
                jobs.append((i, "a", x, us[i], True))
            if ctx.needs_input_grad[4 + 3 * i]:
                jobs.append((i, "b", grads[i], lora[i][2], False))
        wgrads = {}
        if jobs:
            res = lora_grad_batch([j[2] for j in jobs], [j[3] for j in jobs], [j[4] for j in jobs])
            for j, r in zip(jobs, res):
                wgrads[(j[0], j[1])] = r
        out = [grad_x, None]
        for i, (g, pr, lo) in enumerate(zip(grads, projs, lora)):
            gb = ga = gbb = None
            if ctx.needs_input_grad[2 + 3 * i] and ctx.bias_dtypes[i] is not None:
                gb = g.reshape(-1, g.shape[-1]).sum(0, dtype=ctx.bias_dtypes[i])
            if lo is not None:
                if (i, "a") in wgrads:
                    ga = wgrads[(i, "a")].to(lo[0].dtype)
                if (i, "b") in wgrads:
                    gbb = wgrads[(i, "b")].to(lo[1].dtype)
            out += [gb, ga, gbb]
        return tuple(out)


def nf4_linear_group(x, projections: Sequence[Projection]):
    """Outputs of all `projections` applied to the same x, computed by one grouped launch."""
    params = []
    for pr in projections:
        if (pr.lora_a is None) != (pr.lora_b is None):
            raise ValueError("a projection needs both LoRA factors or none")
        if pr.lora_a is not None and pr.lora_a.shape[0] != RANK:
            raise ValueError(f"LoRA rank must be {RANK}")
        params += [pr.bias, pr.lora_a, pr.lora_b]
    return NF4LinearGroup.apply(x, list(projections), *params)
