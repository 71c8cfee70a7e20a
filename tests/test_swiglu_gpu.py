"""GPU: SwiGLU, elementwise and fused into the gate / up GEMM's epilogue, through the C ABI,
against the oracle, the reference kernel's golden vectors and the unfused path."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import nf4_oracle
from tests.util import oracle_weight, synthetic_weight

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
TOL = 1e-2          # GEMM outputs: max |err| / max |ref|
ACT_TOL = 2e-3      # the reference's own tolerance for its SwiGLU kernel (solution/test_kernels.py:28-30)


def fp16_steps(a, b):
    return (a.view(torch.int16).int() - b.view(torch.int16).int()).abs()


@pytest.mark.parametrize("name", ["ragged", "blocks"])
def test_elementwise_matches_reference_kernel(cuda_lib, name):
    from hackaton_b200.mlp import swiglu_backward, swiglu_forward

    z = np.load(GOLDEN / "swiglu_small.npz")
    gate, up, dout = (torch.from_numpy(z[f"{name}_{k}"]).cuda() for k in ("gate", "up", "dout"))
    hidden = swiglu_forward(gate, up)
    dgate, dup = swiglu_backward(dout, gate, up)
    for key, val in (("hidden", hidden), ("dgate", dgate), ("dup", dup)):
        want = torch.from_numpy(z[f"{name}_{key}"])
        torch.testing.assert_close(val.cpu().float(), want.float(), rtol=ACT_TOL, atol=ACT_TOL)
        big = want.abs() > 1e-3                     # fp16 steps only mean something off zero
        assert int(fp16_steps(val.cpu(), want)[big].max()) <= 2, key
    cuda_lib.device_status()


@pytest.mark.parametrize("shape", [(4, 512, 8960), (3, 77, 1001)])   # solution/test_kernels.py:12
def test_silu_mul_matches_pytorch(cuda_lib, shape):
    from hackaton_b200.mlp import silu_mul

    g = torch.Generator(device="cuda").manual_seed(0)
    gate = torch.randn(shape, device="cuda", generator=g).half().requires_grad_()
    up = torch.randn(shape, device="cuda", generator=g).half().requires_grad_()
    grad = torch.randn(shape, device="cuda", generator=g).half()
    ref = torch.nn.functional.silu(gate.float()) * up.float()
    ref.backward(grad.float())
    ref_dgate, ref_dup = gate.grad.float(), up.grad.float()
    gate.grad = up.grad = None
    out = silu_mul(gate, up)
    out.backward(grad)
    torch.testing.assert_close(out.float(), ref, rtol=ACT_TOL, atol=ACT_TOL)
    torch.testing.assert_close(gate.grad.float(), ref_dgate, rtol=ACT_TOL, atol=ACT_TOL)
    torch.testing.assert_close(up.grad.float(), ref_dup, rtol=ACT_TOL, atol=ACT_TOL)
    cuda_lib.device_status()


def mlp_case(m, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).half()
    wg = synthetic_weight(n, k, True, seed=seed + 1, device="cuda")
    wu = synthetic_weight(n, k, True, seed=seed + 2, device="cuda")
    return x, wg, wu


@pytest.mark.parametrize("m,k,n", [
    (2048, 1536, 8960),     # gate / up of Qwen2.5-1.5B at the benchmark's token count
    (300, 192, 264),        # ragged rows, a last tile of 8 columns
    (700, 128, 136),        # two row tiles, ragged both ways
    (64, 1536, 256),        # few rows: grouped GEMM + elementwise kernel behind the same call
    (200, 192, 512),
])
def test_gate_up_swiglu_vs_oracle(cuda_lib, m, k, n):
    from hackaton_b200.group import linear_forward_group
    from hackaton_b200.mlp import gate_up_swiglu_forward

    x, wg, wu = mlp_case(m, k, n, seed=m + n)
    xg = x.cuda()
    hidden, gate, up = gate_up_swiglu_forward(xg, wg, wu, keep=True)
    only_hidden, none_g, none_u = gate_up_swiglu_forward(xg, wg, wu, keep=False)
    torch.cuda.synchronize()
    assert none_g is None and none_u is None
    assert torch.equal(hidden, only_hidden)
    gate_ref = nf4_oracle.linear_fwd(x, oracle_weight(*wg), None)
    up_ref = nf4_oracle.linear_fwd(x, oracle_weight(*wu), None)
    assert nf4_oracle.max_rel_err(gate.cpu(), gate_ref) <= TOL
    assert nf4_oracle.max_rel_err(up.cpu(), up_ref) <= TOL
    assert nf4_oracle.max_rel_err(hidden.cpu(), nf4_oracle.swiglu_fwd(gate_ref, up_ref)) <= TOL
    # the product itself, from the values this kernel wrote for gate and up
    torch.testing.assert_close(hidden.cpu().float(), nf4_oracle.swiglu_fwd(gate.cpu(), up.cpu()).float(),
                               rtol=ACT_TOL, atol=ACT_TOL)
    # same contraction order as the grouped launch without the product
    g2, u2 = linear_forward_group(xg, [wg, wu])
    assert nf4_oracle.max_rel_err(gate.cpu(), g2.cpu()) <= 2e-3
    assert nf4_oracle.max_rel_err(up.cpu(), u2.cpu()) <= 2e-3
    cuda_lib.device_status()


@pytest.mark.parametrize("m,k,n", [(1024, 1536, 8960), (300, 192, 264), (100, 256, 384)])
def test_mlp_front_half_autograd(cuda_lib, m, k, n):
    from hackaton_b200 import Projection
    from hackaton_b200.mlp import nf4_gate_up_swiglu

    x, wg, wu = mlp_case(m, k, n, seed=7 * m + n)
    g = torch.Generator().manual_seed(99)
    d_hidden = torch.randn(m, n, generator=g).half()
    xg = x.cuda().requires_grad_()
    hidden = nf4_gate_up_swiglu(xg, Projection(*wg), Projection(*wu))
    hidden.backward(d_hidden.cuda())
    torch.cuda.synchronize()
    w_gate, w_up = oracle_weight(*wg), oracle_weight(*wu)
    gate_ref, up_ref = nf4_oracle.linear_fwd(x, w_gate, None), nf4_oracle.linear_fwd(x, w_up, None)
    assert nf4_oracle.max_rel_err(hidden.detach().cpu(), nf4_oracle.swiglu_fwd(gate_ref, up_ref)) <= TOL
    d_gate, d_up = nf4_oracle.swiglu_bwd(d_hidden, gate_ref, up_ref)
    dx_ref = d_gate.float() @ w_gate.float() + d_up.float() @ w_up.float()
    assert nf4_oracle.max_rel_err(xg.grad.cpu(), dx_ref) <= TOL
    # without autograd the same call writes only `hidden`, with the same bits
    with torch.no_grad():
        again = nf4_gate_up_swiglu(x.cuda(), Projection(*wg), Projection(*wu))
    assert torch.equal(again, hidden.detach())
    cuda_lib.device_status()


@pytest.mark.parametrize("m,n_down,k_down", [
    (2048, 1536, 8960),     # down_proj of Qwen2.5-1.5B: one kernel (512-row tiles, no K-slices)
    (700, 128, 320),        # ragged, still the pair kernel
    (2048, 256, 512),       # few tiles: K-slices, so dX + elementwise kernel behind the same call
    (100, 192, 384),        # few rows
])
def test_down_backward_with_swiglu_epilogue(cuda_lib, m, n_down, k_down):
    from hackaton_b200.mlp import linear_backward_dx_swiglu, swiglu_backward
    from hackaton_b200.nf4 import linear_backward_dx

    g = torch.Generator().manual_seed(m + k_down)
    wd = synthetic_weight(n_down, k_down, True, seed=5, device="cuda")
    dy = torch.randn(m, n_down, generator=g).half()
    gate = torch.randn(m, k_down, generator=g).half()
    up = torch.randn(m, k_down, generator=g).half()
    d_gate, d_up = linear_backward_dx_swiglu(dy.cuda(), wd, gate.cuda(), up.cuda())
    torch.cuda.synchronize()
    w = oracle_weight(*wd)
    d_hidden = (dy.float() @ w.float()).half()
    rg, ru = nf4_oracle.swiglu_bwd(d_hidden, gate, up)
    assert nf4_oracle.max_rel_err(d_gate.cpu(), rg) <= TOL
    assert nf4_oracle.max_rel_err(d_up.cpu(), ru) <= TOL
    # against the two-step form on the GPU: the same d_hidden bits go into the same arithmetic
    dh = linear_backward_dx(dy.cuda(), wd[0], wd[1])
    g2, u2 = swiglu_backward(dh, gate.cuda(), up.cuda())
    assert nf4_oracle.max_rel_err(d_gate.cpu(), g2.cpu()) <= 2e-3
    assert nf4_oracle.max_rel_err(d_up.cpu(), u2.cpu()) <= 2e-3
    cuda_lib.device_status()


@pytest.mark.parametrize("m,hidden,inter", [(1024, 1536, 8960), (300, 192, 320), (64, 256, 512)])
def test_whole_mlp_autograd(cuda_lib, m, hidden, inter):
    from hackaton_b200 import Projection
    from hackaton_b200.mlp import nf4_swiglu_mlp

    x, wg, wu = mlp_case(m, hidden, inter, seed=3 * m + inter)
    wd = synthetic_weight(hidden, inter, True, seed=17, device="cuda")
    g = torch.Generator().manual_seed(123)
    dy = torch.randn(m, hidden, generator=g).half()
    xg = x.cuda().requires_grad_()
    y = nf4_swiglu_mlp(xg, Projection(*wg), Projection(*wu), Projection(*wd))
    y.backward(dy.cuda())
    torch.cuda.synchronize()
    w_gate, w_up, w_down = oracle_weight(*wg), oracle_weight(*wu), oracle_weight(*wd)
    gate_ref, up_ref = nf4_oracle.linear_fwd(x, w_gate, None), nf4_oracle.linear_fwd(x, w_up, None)
    h_ref = nf4_oracle.swiglu_fwd(gate_ref, up_ref)
    y_ref = nf4_oracle.linear_fwd(h_ref, w_down, None)
    assert nf4_oracle.max_rel_err(y.detach().cpu(), y_ref) <= TOL
    d_hidden = (dy.float() @ w_down.float()).half()
    d_gate, d_up = nf4_oracle.swiglu_bwd(d_hidden, gate_ref, up_ref)
    dx_ref = d_gate.float() @ w_gate.float() + d_up.float() @ w_up.float()
    assert nf4_oracle.max_rel_err(xg.grad.cpu(), dx_ref) <= TOL
    cuda_lib.device_status()
