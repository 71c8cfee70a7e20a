"""GPU: the allocation-free forward entry point (`nf4b200_linear_fwd_static`) against the regular
one (`nf4b200_linear_fwd` with a caller-owned workspace) and against the CPU oracle, through the
C ABI.

Who needs it: callers that cannot give the library device memory, for example a server whose
memory pool is fully assigned at start-up or a plug-in that may not allocate inside its host's
stream-ordered region. Their split-K scratch is a fixed array inside the library; the call itself
allocates nothing. The file sorts last so that a run that stops at the first failure has already
been through every other test.
"""

import ctypes

import pytest
import torch

from oracle import nf4_oracle
from tests.util import oracle_weight, synthetic_weight

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _ptr(t):
    return None if t is None else t.data_ptr()


def _call(lib_mod, fn_name, ref, x, y, workspace=None, bias=None, xa=None, lora_b=None):
    lib = lib_mod.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if fn_name == "static":
        rc = lib.nf4b200_linear_fwd_static(ctypes.byref(ref.struct), x.data_ptr(), x.shape[0],
                                           x.stride(0), _ptr(bias), _ptr(xa), _ptr(lora_b),
                                           y.data_ptr(), y.stride(0), stream)
    else:
        rc = lib.nf4b200_linear_fwd(ctypes.byref(ref.struct), x.data_ptr(), x.shape[0],
                                    x.stride(0), _ptr(bias), _ptr(xa), _ptr(lora_b), y.data_ptr(),
                                    y.stride(0), _ptr(workspace),
                                    0 if workspace is None else workspace.numel(), stream)
    lib_mod.check(rc)


def test_static_scratch_forward_matches_regular_entry_point(cuda_lib):
    from hackaton_b200.nf4 import weight_ref

    n, k, m = 1536, 8960, 300            # a split-K shape: 6 tiles, 140 k-blocks
    packed, state = synthetic_weight(n, k, True, seed=21, device="cuda")
    ref = weight_ref(packed.reshape(-1), state)
    need = cuda_lib.lib().nf4b200_workspace_bytes(n, k, m, 0)
    assert 0 < need <= cuda_lib.STATIC_SCRATCH_BYTES
    workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
    w = oracle_weight(packed, state)
    g = torch.Generator(device="cuda").manual_seed(5)
    for call in range(2):                # two calls in a row share the built-in array
        x = torch.randn(m, k, generator=g, device="cuda").half()
        want = torch.empty(m, n, dtype=torch.float16, device="cuda")
        got = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        _call(cuda_lib, "regular", ref, x, want, workspace)
        _call(cuda_lib, "static", ref, x, got)
        torch.cuda.synchronize()
        err = nf4_oracle.max_rel_err(got.cpu(), nf4_oracle.linear_fwd(x.cpu(), w))
        assert err <= TOL, f"call {call}: max rel err against the oracle {err}"
        assert torch.equal(got, want), f"call {call}: same kernels, same slice order"
    assert cuda_lib.device_status() == 0


@pytest.mark.parametrize("m,n,k", [(16, 1536, 1536),     # a few token rows: the weight-streaming kernel
                                   (300, 512, 1536),     # split-K scratch in use, bias and LoRA on
                                   (2048, 8960, 1536)])  # enough tiles: no scratch at all
def test_static_scratch_allocates_nothing_and_matches_the_oracle(cuda_lib, m, n, k):
    """Bias and the rank-16 term through the allocation-free entry point, for a shape of each
    route, against the oracle; after one warm-up call (which loads the library's device image
    with its built-in array) a call changes neither the free device memory nor torch's own
    allocation count."""
    from hackaton_b200.nf4 import weight_ref

    packed, state = synthetic_weight(n, k, True, seed=23 + m, device="cuda")
    ref = weight_ref(packed.reshape(-1), state).prepare()
    w = oracle_weight(packed, state)
    g = torch.Generator().manual_seed(6)
    x = torch.randn(m, k, generator=g).half()
    bias = torch.randn(n, generator=g).half()
    a = ((torch.rand(16, k, generator=g) * 2 - 1) / k ** 0.5).half()
    b = (torch.randn(n, 16, generator=g) * 0.1).half()
    xa = (2.0 * (x.float() @ a.float().t())).half()          # scaling * x . A^T, as the kernel takes it
    x_d, bias_d, xa_d, b_d = (t.cuda() for t in (x, bias, xa, b))
    y = torch.empty(m, n, dtype=torch.float16, device="cuda")
    _call(cuda_lib, "static", ref, x_d, y, bias=bias_d, xa=xa_d, lora_b=b_d)   # warm-up
    torch.cuda.synchronize()
    # Device-wide free memory can move for reasons outside this process' calls (the driver's own
    # housekeeping), so the measurement is repeated: a call that allocated would show every time.
    unchanged = False
    for _ in range(3):
        free0, used0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        y.fill_(float("nan"))
        _call(cuda_lib, "static", ref, x_d, y, bias=bias_d, xa=xa_d, lora_b=b_d)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == used0
        if torch.cuda.mem_get_info()[0] >= free0:
            unchanged = True
            break
    assert unchanged, "free device memory shrank on every one of three calls"
    want = (x.float() @ w.float().t() + bias.float() + xa.float() @ b.float().t()).half()
    assert nf4_oracle.max_rel_err(y.cpu(), want) <= TOL
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
