"""NF4 decode and the frozen-weight 4-bit linear on B200, behind the reference's Python surface.

Same names, arguments and meaning as the reference's solution/nf4.py:
`can_dequantize(packed, state)`, `dequantize_nf4(packed, state)`, `NF4Linear`,
`nf4_linear(x, packed, bias, state)`. Differences, all in the direction of doing more on the GPU:

* double-quantised states (`state.nested == True`: uint8 absmax + `state.state2` + `state.offset`)
  are accepted directly; the reference needs them flattened to fp32 first
  (solution/packed.py:57-79);
* `NF4Linear` never materialises the fp16 weight: decode is fused into the tcgen05 GEMM, forward
  (x . Wᵀ) and backward (dy . W);
* unsupported input raises instead of silently taking another path (there is none).
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

_DTYPE_CODE = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}


def _numel(shape):
    n = 1
    for d in shape:
        n *= int(d)
    return n


def can_dequantize(packed, state):
    """True when `dequantize_nf4` / `nf4_linear` accept this weight (solution/nf4.py:54-64,
    widened to nested states)."""
    absmax = getattr(state, "absmax", None)
    code = getattr(state, "code", None)
    blocksize = getattr(state, "blocksize", 0)
    shape = getattr(state, "shape", None)
    if not (isinstance(packed, torch.Tensor) and packed.is_cuda and packed.dtype == torch.uint8
            and getattr(state, "quant_type", None) == "nf4" and shape is not None
            and isinstance(absmax, torch.Tensor) and absmax.is_cuda
            and isinstance(code, torch.Tensor) and code.numel() == 16
            and blocksize > 0 and blocksize % 8 == 0
            and packed.numel() * 2 == _numel(shape) and _numel(shape) % 8 == 0
            and _numel(shape) % blocksize == 0
            and packed.is_contiguous() and packed.data_ptr() % 4 == 0
            and getattr(state, "dtype", None) in _DTYPE_CODE):
        return False
    if getattr(state, "nested", False):
        state2 = getattr(state, "state2", None)
        offset = getattr(state, "offset", None)
        return (absmax.dtype == torch.uint8 and state2 is not None and offset is not None
                and isinstance(getattr(state2, "absmax", None), torch.Tensor)
                and isinstance(getattr(state2, "code", None), torch.Tensor)
                and state2.code.numel() == 256 and getattr(state2, "blocksize", 0) > 0)
    return absmax.dtype == torch.float32


# Fused GEMM calls fetch ready-made fp16 block scales (built once per weight) instead of gathering
# absmax / absmax2 on every call. Same results bit for bit; NF4B200_NO_PREPARED=1 turns it off.
PREPARED_SCALES = os.environ.get("NF4B200_NO_PREPARED", "0") != "1"


class WeightRef:
    """The C descriptor of one quantised weight plus the tensors it points into (kept alive)."""

    def __init__(self, packed, state):
        device = packed.device
        rows, cols = (int(state.shape[0]), int(state.shape[1])) if len(state.shape) == 2 else \
            (1, _numel(state.shape))
        keep = [packed]

        def f32(t):
            if not isinstance(t, torch.Tensor):
                t = torch.tensor(float(t))
            t = t.detach()
            if t.device != device or t.dtype != torch.float32 or not t.is_contiguous():
                t = t.to(device=device, dtype=torch.float32).contiguous()
            keep.append(t)
            return t

        code16 = f32(state.code)
        nested = bool(getattr(state, "nested", False))
        w = _lib.Weight()
        w.codes = packed.data_ptr()
        w.code16 = code16.data_ptr()
        w.n_rows, w.n_cols = rows, cols
        w.blocksize = int(state.blocksize)
        w.nested = int(nested)
        if nested:
            absmax = state.absmax.contiguous()
            keep.append(absmax)
            w.absmax = absmax.data_ptr()
            w.code2 = f32(state.state2.code).data_ptr()
            w.absmax2 = f32(state.state2.absmax).data_ptr()
            w.offset = f32(state.offset).reshape(1).data_ptr()
            w.nested_blocksize = int(state.state2.blocksize)
        else:
            w.absmax = f32(state.absmax).data_ptr()
            w.nested_blocksize = 1
        self.struct = w
        self.keep = keep
        self.key = _content_key(packed, state)
        self.rows, self.cols = rows, cols
        self.scales16 = None
        self._ready = None   # (event, stream) of the table's construction while it may be pending

    def prepare(self):
        """Builds, once, the fp16 block-scale table the fused GEMM can fetch by TMA (see
        nf4b200_prepare_scales in include/nf4b200.h) and hooks it into the descriptor. Weights
        are frozen in QLoRA, so the table stays valid while the state's tensors are not written
        (`weight_ref` drops the descriptor when they are). No host synchronisation: a call on
        another stream than the one that built the table waits for the build on the device.
        Under CUDA-graph capture nothing can wait on work outside the capture, so build the
        tables (`prepare_weights`) and let them finish before capturing."""
        if self.scales16 is not None or not PREPARED_SCALES:
            if self._ready is not None:
                self._order_after_build()
            return self
        need = int(_lib.lib().nf4b200_scales16_bytes(self.rows, self.cols))
        if need == 0 or self.struct.blocksize != 64:
            return self
        device = self.keep[0].device
        table = torch.empty(need // 2, dtype=torch.float16, device=device)
        with torch.cuda.device(device):
            _lib.check(_lib.lib().nf4b200_prepare_scales(ctypes.byref(self.struct), table.data_ptr(),
                                                         _stream_ptr(device)))
            if not torch.cuda.is_current_stream_capturing():
                event = torch.cuda.Event()
                event.record()
                self._ready = (event, torch.cuda.current_stream(device).cuda_stream)
        self.scales16 = table
        self.struct.scales16 = table.data_ptr()
        return self

    def _order_after_build(self):
        if torch.cuda.is_current_stream_capturing():
            return   # a capture cannot wait on outside work: build the tables before capturing
        event, stream = self._ready
        current = torch.cuda.current_stream(self.keep[0].device)
        if event.query():
            self._ready = None
            return
        if current.cuda_stream != stream:
            current.wait_event(event)


def _content_key(packed, state):
    """Identity of a weight's contents: where its tensors live and how often they have been
    written in place. Loading other weights into the same storage (`copy_`, a second checkpoint)
    bumps the version counters, so a cached descriptor (and its scale table) is not reused."""
    nested = bool(getattr(state, "nested", False))
    parts = [packed.data_ptr(), packed._version, state.absmax.data_ptr(), state.absmax._version,
             nested]
    if nested:
        state2 = state.state2
        offset = state.offset
        parts += [state2.absmax.data_ptr(), state2.absmax._version,
                  offset._version if isinstance(offset, torch.Tensor) else float(offset)]
    return tuple(parts)


def prepare_weights(weights):
    """Builds the scale tables of many weights back to back (a whole model's at load time):
    `weights` is an iterable of (packed, state). Nothing waits on the host; returns the
    descriptors."""
    return [weight_ref(packed.reshape(-1), state).prepare() for packed, state in weights]


def weight_ref(packed, state) -> WeightRef:
    """Descriptor for (packed, state), cached on the state object while its tensors stay put and
    unwritten."""
    cached = getattr(state, "_nf4b200_ref", None)
    if cached is not None and cached.key == _content_key(packed, state):
        return cached
    ref = WeightRef(packed, state)
    try:
        state._nf4b200_ref = ref
    except AttributeError:  # states with __slots__: build the descriptor per call
        pass
    return ref


def _stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_ws_need = {}      # (device, n_rows, n_cols, m, backward) -> bytes of split-K scratch
_ws_buffers = {}   # (device, stream) -> uint8 tensor


def _workspace(device, n_rows, n_cols, m, backward):
    """Split-K scratch for one GEMM call on the current stream: (pointer, bytes) or (None, 0).
    One buffer per (device, stream), grown on demand; it needs no initialisation. Calls on the
    same stream run one after the other and can share it; other streams get their own."""
    key = (device.index, n_rows, n_cols, m, backward)
    need = _ws_need.get(key)
    if need is None:
        with torch.cuda.device(device):
            need = int(_lib.lib().nf4b200_workspace_bytes(n_rows, n_cols, m, int(backward)))
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


def _require(packed, state):
    if not can_dequantize(packed, state):
        raise ValueError(
            "hackaton_b200: unsupported NF4 weight (needs a contiguous CUDA uint8 tensor of NF4 "
            "codes and a quant state with fp32 absmax, or uint8 absmax + state2 + offset)")


def dequantize_nf4(packed, state):
    """The weight `state.shape` in `state.dtype` from its packed NF4 bytes
    (solution/nf4.py:67-77); bit-equal to the reference's decode."""
    packed = packed.reshape(-1)
    _require(packed, state)
    ref = weight_ref(packed, state)
    out = torch.empty(tuple(state.shape), dtype=state.dtype, device=packed.device)
    with torch.cuda.device(packed.device):
        _lib.check(_lib.lib().nf4b200_dequant(ctypes.byref(ref.struct), out.data_ptr(),
                                              _DTYPE_CODE[state.dtype], _stream_ptr(packed.device)))
    return out


def _rows_view(t, cols):
    """[..., cols] -> contiguous-row 2-D view (copying only if the layout forces it)."""
    t2 = t.reshape(-1, cols)
    if t2.stride(1) != 1 or t2.stride(0) % 8 != 0 or t2.data_ptr() % 16 != 0 or \
            (t2.shape[0] > 1 and t2.stride(0) < cols):
        t2 = t2.contiguous()
    return t2


def linear_forward(x, packed, bias, state, xa=None, lora_b=None):
    """y = x . Wᵀ (+ bias) (+ xa . lora_bᵀ) through the fused kernel. x: fp16 [..., K]."""
    packed = packed.reshape(-1)
    _require(packed, state)
    ref = weight_ref(packed, state).prepare()
    if x.dtype != torch.float16:
        raise TypeError(f"hackaton_b200: the fused NF4 linear computes in fp16, got {x.dtype}")
    if x.shape[-1] != ref.cols:
        raise ValueError(f"input has {x.shape[-1]} features, weight expects {ref.cols}")
    x2 = _rows_view(x, ref.cols)
    m = x2.shape[0]
    y = torch.empty((m, ref.rows), dtype=torch.float16, device=x.device)
    if m == 0:
        return y.reshape(*x.shape[:-1], ref.rows)
    if bias is not None:
        bias = bias.to(torch.float16).contiguous()
    ws, ws_bytes = _workspace(x.device, ref.rows, ref.cols, m, False)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().nf4b200_linear_fwd(
            ctypes.byref(ref.struct), x2.data_ptr(), m, x2.stride(0),
            None if bias is None else bias.data_ptr(),
            None if xa is None else xa.data_ptr(), None if lora_b is None else lora_b.data_ptr(),
            y.data_ptr(), y.stride(0), ws, ws_bytes, _stream_ptr(x.device)))
    return y.reshape(*x.shape[:-1], ref.rows)


def linear_backward_dx(grad_output, packed, state, u=None, lora_a=None):
    """dx = dy . W (+ u . lora_a) through the fused kernel. dy: fp16 [..., N]."""
    packed = packed.reshape(-1)
    _require(packed, state)
    ref = weight_ref(packed, state).prepare()
    if grad_output.dtype != torch.float16:
        raise TypeError(f"hackaton_b200: the fused NF4 linear computes in fp16, got {grad_output.dtype}")
    g2 = _rows_view(grad_output, ref.rows)
    m = g2.shape[0]
    dx = torch.empty((m, ref.cols), dtype=torch.float16, device=grad_output.device)
    if m == 0:
        return dx.reshape(*grad_output.shape[:-1], ref.cols)
    ws, ws_bytes = _workspace(grad_output.device, ref.rows, ref.cols, m, True)
    with torch.cuda.device(grad_output.device):
        _lib.check(_lib.lib().nf4b200_linear_bwd_dx(
            ctypes.byref(ref.struct), g2.data_ptr(), m, g2.stride(0),
            None if u is None else u.data_ptr(), None if lora_a is None else lora_a.data_ptr(),
            dx.data_ptr(), dx.stride(0), ws, ws_bytes, _stream_ptr(grad_output.device)))
    return dx.reshape(*grad_output.shape[:-1], ref.cols)


class NF4Linear(torch.autograd.Function):
    """x @ Wᵀ + bias for a frozen NF4 weight W (solution/nf4.py:80-102), with the decode fused
    into the matrix product in both directions. Nothing but the packed bytes and their quant
    state is kept for the backward pass."""

    @staticmethod
    def forward(ctx, x, packed, bias, state):
        ctx.packed, ctx.state = packed, state
        ctx.bias_dtype = None if bias is None else bias.dtype
        return linear_forward(x, packed, bias, state)

    @staticmethod
    def backward(ctx, grad_output):
        grad_x = grad_bias = None
        if ctx.needs_input_grad[0]:
            grad_x = linear_backward_dx(grad_output, ctx.packed, ctx.state)
        if ctx.needs_input_grad[2]:
            grad_bias = grad_output.reshape(-1, grad_output.shape[-1]).sum(0, dtype=ctx.bias_dtype)
        return grad_x, None, grad_bias, None


def nf4_linear(x, packed, bias, state):
    return NF4Linear.apply(x, packed.reshape(-1), bias, state)
