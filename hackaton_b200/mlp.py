"""SwiGLU next to the gate / up projections: the step right after the two biggest NF4 GEMMs.

The reference runs `silu_mul(gate_proj(x16), up_proj(x16))` (solution/patches.py:39-41) with an
elementwise Triton kernel (`silu_mul_kernel` / `SiluMul`, solution/kernels.py:39-96) that reads
the two [tokens, 8960] fp16 arrays back from memory. Here:

* `silu_mul(gate, up)`: the same function on the library's own elementwise kernels (forward and
  backward), fp32 arithmetic with one rounding, keeps gate and up for the backward pass.
* `nf4_gate_up_swiglu(x, gate_proj, up_proj)`: both projections AND the product in one kernel:
  the product is formed while the accumulators are drained. Under autograd gate and up are
  written as well (the backward needs them, as in the reference); without it only `hidden`
  leaves the chip. Backward: one elementwise kernel (d_gate, d_up), then one grouped dX GEMM.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .group import Projection, _refs, linear_backward_dx_group
from .nf4 import _rows_view, _stream_ptr, _ws_buffers

_ws_need = {}


def swiglu_forward(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """hidden = silu(gate) * up on fp16 CUDA tensors of the same shape."""
    _check_pair(gate, up)
    gate, up = gate.contiguous(), up.contiguous()
    out = torch.empty_like(gate)
    with torch.cuda.device(gate.device):
        _lib.check(_lib.lib().nf4b200_swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(),
                                                 gate.numel(), _stream_ptr(gate.device)))
    return out


def swiglu_backward(d_hidden: torch.Tensor, gate: torch.Tensor, up: torch.Tensor):
    """(d_gate, d_up) for hidden = silu(gate) * up."""
    _check_pair(gate, up)
    _check_pair(d_hidden, gate)
    d_hidden, gate, up = d_hidden.contiguous(), gate.contiguous(), up.contiguous()
    d_gate, d_up = torch.empty_like(gate), torch.empty_like(up)
    with torch.cuda.device(gate.device):
        _lib.check(_lib.lib().nf4b200_swiglu_bwd(
            d_hidden.data_ptr(), gate.data_ptr(), up.data_ptr(), d_gate.data_ptr(), d_up.data_ptr(),
            gate.numel(), _stream_ptr(gate.device)))
    return d_gate, d_up


def _check_pair(a, b):
    if a.dtype != torch.float16 or b.dtype != torch.float16:
        raise TypeError(f"hackaton_b200: SwiGLU computes on fp16 tensors, got {a.dtype}, {b.dtype}")
    if a.shape != b.shape:
        raise ValueError(f"hackaton_b200: SwiGLU operands differ in shape: {tuple(a.shape)}, {tuple(b.shape)}")
    if not (a.is_cuda and b.is_cuda):
        raise ValueError("hackaton_b200: SwiGLU needs CUDA tensors (there is no CPU path)")


class SiluMul(torch.autograd.Function):
    """silu(gate) * up; keeps gate and up (fp16) for the backward, like the reference's SiluMul
    (solution/kernels.py:60-91) without its host-offload option."""

    @staticmethod
    def forward(ctx, gate, up):
        ctx.save_for_backward(gate, up)
        return swiglu_forward(gate, up)

    @staticmethod
    def backward(ctx, d_hidden):
        gate, up = ctx.saved_tensors
        return swiglu_backward(d_hidden, gate, up)


def silu_mul(gate, up):
    """solution/kernels.py:94-96."""
    return SiluMul.apply(gate, up)


def _workspace(device, rows, cols, m, keep):
    key = (device.index, rows, cols, m, keep)
    need = _ws_need.get(key)
    if need is None:
        with torch.cuda.device(device):
            need = int(_lib.lib().nf4b200_gate_up_swiglu_workspace_bytes(rows, cols, m, int(keep)))
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
    return buf.data_ptr(), need


def gate_up_swiglu_forward(x, gate_w, up_w, keep: bool):
    """gate_w, up_w: (packed, state). Returns (hidden, gate, up); gate and up are None unless
    `keep`. One kernel for more than 256 token rows (see nf4b200_gate_up_swiglu_fwd)."""
    refs = _refs([gate_w, up_w])
    if refs[0].rows != refs[1].rows:
        raise ValueError("hackaton_b200: gate and up projections differ in shape")
    if x.dtype != torch.float16:
        raise TypeError(f"hackaton_b200: the fused NF4 linear computes in fp16, got {x.dtype}")
    rows, cols = refs[0].rows, refs[0].cols
    x2 = _rows_view(x, cols)
    m = x2.shape[0]
    lead = x.shape[:-1]
    hidden = torch.empty((m, rows), dtype=torch.float16, device=x.device)
    gate = torch.empty_like(hidden) if keep else None
    up = torch.empty_like(hidden) if keep else None
    if m > 0:
        ws, ws_bytes = _workspace(x.device, rows, cols, m, keep)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().nf4b200_gate_up_swiglu_fwd(
                ctypes.byref(refs[0].struct), ctypes.byref(refs[1].struct), x2.data_ptr(), m,
                x2.stride(0), None if gate is None else gate.data_ptr(),
                None if up is None else up.data_ptr(), hidden.data_ptr(), ws, ws_bytes,
                _stream_ptr(x.device)))
    shape = (*lead, rows)
    return (hidden.reshape(shape), None if gate is None else gate.reshape(shape),
            None if up is None else up.reshape(shape))


class NF4GateUpSwiGLU(torch.autograd.Function):
    """hidden = silu(x . Wgᵀ) * (x . Wuᵀ) for two frozen NF4 weights; gradient flows to x."""

    @staticmethod
    def forward(ctx, x, gate_w, up_w):
        keep = ctx.needs_input_grad[0]
        hidden, gate, up = gate_up_swiglu_forward(x, gate_w, up_w, keep)
        if keep:
            ctx.save_for_backward(gate, up)
            ctx.weights = (gate_w, up_w)
        return hidden

    @staticmethod
    def backward(ctx, d_hidden):
        gate, up = ctx.saved_tensors
        d_gate, d_up = swiglu_backward(d_hidden, gate, up)
        dx = linear_backward_dx_group([d_gate, d_up], list(ctx.weights))
        return dx, None, None


def linear_backward_dx_swiglu(grad_out, down_w, gate, up):
    """(d_gate, d_up) from the gradient of down_proj's output: d_hidden = grad_out . W_down never
    reaches memory when the plan allows it (see nf4b200_linear_bwd_dx_swiglu). down_w: (packed,
    state); gate, up: what the forward kept, [..., K_down] fp16."""
    ref = _refs([down_w])[0]
    _check_pair(gate, up)
    if grad_out.dtype != torch.float16:
        raise TypeError(f"hackaton_b200: the fused NF4 linear computes in fp16, got {grad_out.dtype}")
    g2 = _rows_view(grad_out, ref.rows)
    m = g2.shape[0]
    gate, up = gate.contiguous(), up.contiguous()
    if gate.numel() != m * ref.cols:
        raise ValueError("hackaton_b200: gate / up do not match the gradient's rows and the weight's columns")
    d_gate, d_up = torch.empty_like(gate), torch.empty_like(up)
    if m == 0:
        return d_gate, d_up
    device = g2.device
    key = (device.index, "bwd", ref.rows, ref.cols, m)
    need = _ws_need.get(key)
    if need is None:
        with torch.cuda.device(device):
            need = int(_lib.lib().nf4b200_linear_bwd_dx_swiglu_workspace_bytes(ref.rows, ref.cols, m))
        if need < 0:
            _lib.check(need)
        _ws_need[key] = need
    ws, ws_bytes = None, 0
    if need:
        skey = (device.index, torch.cuda.current_stream(device).cuda_stream)
        buf = _ws_buffers.get(skey)
        if buf is None or buf.numel() < need:
            buf = torch.empty(max(need, 1 << 22), dtype=torch.uint8, device=device)
            _ws_buffers[skey] = buf
        ws, ws_bytes = buf.data_ptr(), need
    with torch.cuda.device(device):
        _lib.check(_lib.lib().nf4b200_linear_bwd_dx_swiglu(
            ctypes.byref(ref.struct), g2.data_ptr(), m, g2.stride(0), gate.data_ptr(), up.data_ptr(),
            d_gate.data_ptr(), d_up.data_ptr(), ws, ws_bytes, _stream_ptr(device)))
    return d_gate, d_up


class NF4SwiGLUMLP(torch.autograd.Function):
    """y = (silu(x . Wgᵀ) * (x . Wuᵀ)) . Wdᵀ on three frozen NF4 weights: two kernels forward
    (gate/up/product, down), two backward (down's dX with the SwiGLU backward in its epilogue,
    then the grouped dX of gate and up). Keeps gate and up for the backward, not the product."""

    @staticmethod
    def forward(ctx, x, gate_w, up_w, down_w):
        from .nf4 import linear_forward
        keep = ctx.needs_input_grad[0]
        hidden, gate, up = gate_up_swiglu_forward(x, gate_w, up_w, keep)
        y = linear_forward(hidden, down_w[0], None, down_w[1])
        if keep:
            ctx.save_for_backward(gate, up)
            ctx.weights = (gate_w, up_w, down_w)
        return y

    @staticmethod
    def backward(ctx, grad_out):
        gate, up = ctx.saved_tensors
        gate_w, up_w, down_w = ctx.weights
        d_gate, d_up = linear_backward_dx_swiglu(grad_out.contiguous(), down_w, gate, up)
        dx = linear_backward_dx_group([d_gate, d_up], [gate_w, up_w])
        return dx, None, None, None


def nf4_swiglu_mlp(x, gate_proj: Projection, up_proj: Projection, down_proj: Projection):
    """The whole SwiGLU MLP of a Qwen2 block (solution/patches.py:32-41) on NF4 weights without
    bias or LoRA pairs; other configurations go through `nf4_gate_up_swiglu` and the ordinary
    linear."""
    projs = (gate_proj, up_proj, down_proj)
    if all(p.bias is None and p.lora_a is None and p.lora_b is None for p in projs):
        return NF4SwiGLUMLP.apply(x, *[(p.packed, p.state) for p in projs])
    from .lora import nf4_lora_linear
    from .nf4 import nf4_linear
    hidden = nf4_gate_up_swiglu(x, gate_proj, up_proj)
    d = down_proj
    if d.lora_a is not None:
        return nf4_lora_linear(hidden, d.packed, d.bias, d.state, d.lora_a, d.lora_b, d.scaling)
    return nf4_linear(hidden, d.packed, d.bias, d.state)


def nf4_gate_up_swiglu(x, gate_proj: Projection, up_proj: Projection):
    """The front half of a SwiGLU MLP on NF4 weights. Projections with a bias or a LoRA pair are
    not covered by the fused kernel: they take the grouped launch followed by `silu_mul`."""
    plain = all(p.bias is None and p.lora_a is None and p.lora_b is None for p in (gate_proj, up_proj))
    if not plain:
        from .group import nf4_linear_group
        gate, up = nf4_linear_group(x, [gate_proj, up_proj])
        return silu_mul(gate, up)
    return NF4GateUpSwiGLU.apply(x, (gate_proj.packed, gate_proj.state),
                                 (up_proj.packed, up_proj.state))
