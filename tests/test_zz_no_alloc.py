"""GPU: the allocation-free forward entry point (`nf4b200_linear_fwd_static`) against the regular
one (`nf4b200_linear_fwd` with a caller-owned workspace), through the C ABI.

Who needs it: callers that cannot give the library device memory, for example a server whose
memory pool is fully assigned at start-up or a plug-in that may not allocate inside its host's
stream-ordered region. Their split-K scratch is a fixed array inside the library; the call itself
allocates nothing. The file sorts last so that a run that stops at the first failure has already
been through every other test.
"""

import ctypes

import pytest
import torch

from tests.util import synthetic_weight

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _call(lib_mod, fn_name, ref, x, y, workspace=None):
    lib = lib_mod.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if fn_name == "static":
        rc = lib.nf4b200_linear_fwd_static(ctypes.byref(ref.struct), x.data_ptr(), x.shape[0],
                                           x.stride(0), None, None, None, y.data_ptr(),
                                           y.stride(0), stream)
    else:
        rc = lib.nf4b200_linear_fwd(ctypes.byref(ref.struct), x.data_ptr(), x.shape[0],
                                    x.stride(0), None, None, None, y.data_ptr(), y.stride(0),
                                    workspace.data_ptr(), workspace.numel(), stream)
    lib_mod.check(rc)


def test_static_scratch_forward_matches_regular_entry_point(cuda_lib):
    from hackaton_b200.nf4 import weight_ref

    n, k, m = 1536, 8960, 300            # a split-K shape: 6 tiles, 140 k-blocks
    packed, state = synthetic_weight(n, k, True, seed=21, device="cuda")
    ref = weight_ref(packed.reshape(-1), state)
    need = cuda_lib.lib().nf4b200_workspace_bytes(n, k, m, 0)
    assert 0 < need <= cuda_lib.STATIC_SCRATCH_BYTES
    workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    for call in range(2):                # two calls in a row share the built-in array
        x = torch.randn(m, k, generator=g, device="cuda").half()
        want = torch.empty(m, n, dtype=torch.float16, device="cuda")
        got = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        _call(cuda_lib, "regular", ref, x, want, workspace)
        _call(cuda_lib, "static", ref, x, got)
        torch.cuda.synchronize()
        err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
        assert err <= TOL, f"call {call}: max rel err {err}"
        assert torch.equal(got, want), f"call {call}: same kernels, same slice order"
    assert cuda_lib.device_status() == 0


def test_static_scratch_rejects_shapes_beyond_its_size(cuda_lib):
    from hackaton_b200.nf4 import weight_ref

    n, k, m = 1536, 8960, 2048           # 3 slices of 2048 x 1536 fp32: more than the array holds
    need = cuda_lib.lib().nf4b200_workspace_bytes(n, k, m, 0)
    assert need > cuda_lib.STATIC_SCRATCH_BYTES
    packed, state = synthetic_weight(n, k, True, seed=22, device="cuda")
    ref = weight_ref(packed.reshape(-1), state)
    x = torch.zeros(m, k, dtype=torch.float16, device="cuda")
    y = torch.empty(m, n, dtype=torch.float16, device="cuda")
    with pytest.raises(cuda_lib.Nf4Error) as info:
        _call(cuda_lib, "static", ref, x, y)
    assert "scratch" in str(info.value)
