"""ctypes binding of libnf4b200.so (the C ABI declared in include/nf4b200.h).

There is no fallback: if the library has not been built, or the device is not sm_100, every
entry point raises.
"""

from __future__ import annotations

import ctypes
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t,
                    c_void_p)
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libnf4b200.so"

EXPORTS = (
    "nf4b200_query", "nf4b200_last_error", "nf4b200_device_status", "nf4b200_dequant",
    "nf4b200_linear_fwd", "nf4b200_linear_bwd_dx", "nf4b200_lora_down", "nf4b200_lora_grad",
    "nf4b200_workspace_bytes", "nf4b200_linear_fwd_static", "nf4b200_linear_fwd_group",
    "nf4b200_linear_bwd_dx_group", "nf4b200_workspace_bytes_group", "nf4b200_launches_group", "nf4b200_scales16_bytes",
    "nf4b200_prepare_scales", "nf4b200_lora_down_batch", "nf4b200_lora_grad_batch",
    "nf4b200_set_sm_limit", "nf4b200_gate_up_swiglu_fwd", "nf4b200_gate_up_swiglu_workspace_bytes",
    "nf4b200_swiglu_fwd", "nf4b200_swiglu_bwd", "nf4b200_linear_bwd_dx_swiglu",
    "nf4b200_linear_bwd_dx_swiglu_workspace_bytes", "nf4b200_rmsnorm_fwd", "nf4b200_rmsnorm_bwd",
    "nf4b200_qkv_rotate", "nf4b200_ce_stats", "nf4b200_ce_grad", "nf4b200_selftest_wait", "nf4b200_fp16_linear",
)

F16, BF16, F32 = 0, 1, 2
STATIC_SCRATCH_BYTES = 32 << 20   # NF4B200_STATIC_SCRATCH_BYTES in include/nf4b200.h


class Nf4Error(RuntimeError):
    """A non-zero status from the CUDA library."""

    def __init__(self, code: int, message: str):
        super().__init__(f"nf4b200 error {code}: {message}")
        self.code = code


class Weight(Structure):
    _fields_ = [
        ("codes", c_void_p), ("absmax", c_void_p), ("code2", c_void_p), ("absmax2", c_void_p),
        ("offset", c_void_p), ("code16", c_void_p), ("n_rows", c_int64), ("n_cols", c_int64),
        ("blocksize", c_int32), ("nested_blocksize", c_int32), ("nested", c_int32),
        ("reserved", c_int32), ("scales16", c_void_p),
    ]


class Props(Structure):
    _fields_ = [("cc_major", c_int32), ("cc_minor", c_int32), ("sm_count", c_int32),
                ("supported", c_int32), ("smem_per_block_optin", c_int64)]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m hackaton_b200.build` (needs nvcc). "
            "hackaton_b200 has no CPU or PyTorch fallback for its kernels.")
    handle = ctypes.CDLL(str(LIB_PATH))
    handle.nf4b200_last_error.restype = c_char_p
    handle.nf4b200_last_error.argtypes = []
    handle.nf4b200_query.argtypes = [c_int, POINTER(Props)]
    handle.nf4b200_device_status.argtypes = [POINTER(c_int)]
    handle.nf4b200_selftest_wait.argtypes = [c_int64, c_void_p]
    handle.nf4b200_fp16_linear.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64,
                                           c_int64, c_int, c_void_p, c_void_p, c_int64, c_void_p,
                                           c_size_t, c_void_p]
    handle.nf4b200_dequant.argtypes = [POINTER(Weight), c_void_p, c_int, c_void_p]
    handle.nf4b200_linear_fwd.argtypes = [POINTER(Weight), c_void_p, c_int64, c_int64, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                                          c_size_t, c_void_p]
    handle.nf4b200_linear_bwd_dx.argtypes = [POINTER(Weight), c_void_p, c_int64, c_int64, c_void_p,
                                             c_void_p, c_void_p, c_int64, c_void_p, c_size_t,
                                             c_void_p]
    handle.nf4b200_workspace_bytes.argtypes = [c_int64, c_int64, c_int64, c_int]
    handle.nf4b200_linear_fwd_static.argtypes = [POINTER(Weight), c_void_p, c_int64, c_int64,
                                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                                 c_void_p]
    handle.nf4b200_lora_down.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64,
                                         c_int64, c_float, c_void_p, c_void_p]
    handle.nf4b200_lora_grad.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                         c_int64, c_int64, c_void_p]
    pw, pv, pi64 = POINTER(POINTER(Weight)), POINTER(c_void_p), POINTER(c_int64)
    handle.nf4b200_linear_fwd_group.argtypes = [c_int, pw, c_void_p, c_int64, c_int64, pv, pv, pv,
                                                pv, pi64, c_void_p, c_size_t, c_void_p]
    handle.nf4b200_linear_bwd_dx_group.argtypes = [c_int, pw, pv, c_int64, pi64, pv, pv, c_void_p,
                                                   c_int64, c_void_p, c_size_t, c_void_p]
    handle.nf4b200_workspace_bytes_group.argtypes = [c_int, pi64, c_int64, c_int64, c_int]
    handle.nf4b200_workspace_bytes_group.restype = c_int64
    handle.nf4b200_launches_group.argtypes = [c_int, pi64, c_int64, c_int64, c_int, c_int]
    handle.nf4b200_launches_group.restype = c_int
    pf = POINTER(c_float)
    handle.nf4b200_lora_down_batch.argtypes = [c_int, pv, c_int64, pi64, pi64, pv, pi64, pi64, pf,
                                               pv, c_void_p]
    handle.nf4b200_lora_grad_batch.argtypes = [c_int, pv, pi64, pi64, pi64, pv, pv, pi64, pi64,
                                               c_void_p]
    handle.nf4b200_set_sm_limit.argtypes = [c_int]
    handle.nf4b200_scales16_bytes.argtypes = [c_int64, c_int64]
    handle.nf4b200_scales16_bytes.restype = c_int64
    handle.nf4b200_prepare_scales.argtypes = [POINTER(Weight), c_void_p, c_void_p]
    handle.nf4b200_gate_up_swiglu_fwd.argtypes = [POINTER(Weight), POINTER(Weight), c_void_p, c_int64,
                                                  c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                                  c_size_t, c_void_p]
    handle.nf4b200_gate_up_swiglu_workspace_bytes.argtypes = [c_int64, c_int64, c_int64, c_int]
    handle.nf4b200_gate_up_swiglu_workspace_bytes.restype = c_int64
    handle.nf4b200_linear_bwd_dx_swiglu.argtypes = [POINTER(Weight), c_void_p, c_int64, c_int64, c_void_p,
                                                    c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                                    c_void_p]
    handle.nf4b200_linear_bwd_dx_swiglu_workspace_bytes.argtypes = [c_int64, c_int64, c_int64]
    handle.nf4b200_linear_bwd_dx_swiglu_workspace_bytes.restype = c_int64
    handle.nf4b200_rmsnorm_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                           c_void_p, c_int64, c_int64, c_float, c_void_p]
    handle.nf4b200_rmsnorm_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                           c_void_p, c_int64, c_int64, c_void_p]
    handle.nf4b200_qkv_rotate.argtypes = [c_void_p] * 8 + [c_int64, c_int64, c_void_p, c_void_p, c_int64,
                                                           c_int64, c_int, c_int, c_int, c_int, c_int,
                                                           c_int, c_void_p]
    handle.nf4b200_ce_stats.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int64, c_int64, c_void_p]
    handle.nf4b200_ce_grad.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                       c_int64, c_void_p]
    handle.nf4b200_swiglu_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]
    handle.nf4b200_swiglu_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                          c_void_p]
    for name in EXPORTS:
        if name not in ("nf4b200_last_error", "nf4b200_workspace_bytes",
                        "nf4b200_workspace_bytes_group", "nf4b200_scales16_bytes",
                        "nf4b200_gate_up_swiglu_workspace_bytes",
                        "nf4b200_linear_bwd_dx_swiglu_workspace_bytes"):
            getattr(handle, name).restype = c_int
    handle.nf4b200_workspace_bytes.restype = c_int64
    _lib = handle
    return handle


def check(status: int) -> None:
    if status != 0:
        raise Nf4Error(status, lib().nf4b200_last_error().decode("utf-8", "replace"))


def query(device: int = 0) -> Props:
    props = Props()
    check(lib().nf4b200_query(device, ctypes.byref(props)))
    return props


def set_sm_limit(sms: int) -> None:
    """Caps the SMs the fused GEMM grids occupy (0 = all); see nf4b200_set_sm_limit."""
    check(lib().nf4b200_set_sm_limit(int(sms)))
    from . import group, nf4     # scratch sizes were computed for the old grid
    nf4._ws_need.clear()
    group._ws_need.clear()


def device_status() -> int:
    """Reads and clears the device-side status word (synchronises). Raises if it was non-zero."""
    word = c_int(0)
    check(lib().nf4b200_device_status(ctypes.byref(word)))
    return word.value
