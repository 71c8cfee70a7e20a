"""GPU: the fused dequant-GEMM (forward x.Wᵀ, backward dy.W) through the C ABI against the CPU
oracle, at fp16 tolerance: max |err| / max |ref| <= 1e-2 (the bound the task states), and the
reference's own rtol = atol = 2e-3 (solution/test_nf4.py:63-64) where K is small enough for it."""

from pathlib import Path

import numpy as np
import pytest
import torch

from hackaton_b200.quantize import QuantState
from oracle import nf4_oracle
from tests.util import oracle_weight, synthetic_weight

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
TOL = 1e-2


def rel(got, want):
    return nf4_oracle.max_rel_err(got.cpu(), want)


def run_case(m, n, k, nested, bias, seed=0):
    from hackaton_b200 import nf4_linear

    packed, state = synthetic_weight(n, k, nested, seed=seed, device="cuda")
    w = oracle_weight(packed, state)
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(m, k, generator=g).half()
    dy = torch.randn(m, n, generator=g).half()
    b = (torch.randn(n, generator=g) * 0.1).half() if bias else None
    xg = x.cuda().requires_grad_()
    y = nf4_linear(xg, packed.t(), None if b is None else b.cuda(), state)
    y.backward(dy.cuda())
    torch.cuda.synchronize()
    return rel(y, nf4_oracle.linear_fwd(x, w, b)), rel(xg.grad, nf4_oracle.linear_bwd(dy, w))


# (M, N, K): the reference's test shape, tile-aligned and ragged ones, single rows, N < tile
CASES = [(300, 512, 1536), (256, 256, 64), (128, 256, 128), (1, 256, 64), (4, 1536, 1536),
         (77, 100 * 8, 192), (513, 264, 320), (2048, 256, 1536), (130, 8, 64)]


@pytest.mark.parametrize("m,n,k", CASES)
@pytest.mark.parametrize("nested", [True, False])
def test_linear_forward_backward_vs_oracle(cuda_lib, m, n, k, nested):
    ef, eb = run_case(m, n, k, nested, bias=(n % 16 == 0), seed=m + n + k)
    assert ef <= TOL, f"forward max rel err {ef}"
    assert eb <= TOL, f"backward max rel err {eb}"
    cuda_lib.device_status()


def test_config0_q_proj(cuda_lib):
    """One q_proj of the 1.5B model: W[1536,1536], X[2048,1536] (batch 4 x 512 tokens)."""
    ef, eb = run_case(2048, 1536, 1536, True, bias=False, seed=0)
    assert ef <= TOL and eb <= TOL, (ef, eb)


def test_mlp_shapes(cuda_lib):
    """gate/up (8960 <- 1536) and down (1536 <- 8960) at a reduced token count."""
    for n, k in [(8960, 1536), (1536, 8960)]:
        ef, eb = run_case(384, n, k, True, bias=False, seed=n)
        assert ef <= TOL and eb <= TOL, (n, k, ef, eb)


def test_matches_reference_golden_linear(cuda_lib):
    from hackaton_b200 import nf4_linear

    g = np.load(GOLDEN / "linear_small.npz")
    state = QuantState(absmax=torch.from_numpy(g["absmax"]).cuda(),
                       code=torch.from_numpy(g["table"]).cuda(), shape=(96, 192))
    x = torch.from_numpy(g["x"]).cuda().requires_grad_()
    out = nf4_linear(x, torch.from_numpy(g["packed"]).cuda().view(-1, 1).t(),
                     torch.from_numpy(g["bias"]).cuda(), state)
    out.backward(torch.from_numpy(g["grad"]).cuda())
    torch.testing.assert_close(out.detach().cpu(), torch.from_numpy(g["out"]), rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(x.grad.cpu(), torch.from_numpy(g["grad_x"]), rtol=2e-3, atol=2e-3)


def test_leading_dims_and_strided_rows(cuda_lib):
    from hackaton_b200 import nf4_linear

    packed, state = synthetic_weight(256, 128, True, seed=4, device="cuda")
    w = oracle_weight(packed, state)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(3, 50, 256, generator=g).half()
    xs = x.cuda()[..., :128]  # row stride 256, 128 columns used
    y = nf4_linear(xs, packed, None, state)
    assert y.shape == (3, 50, 256)
    assert rel(y.reshape(-1, 256), nf4_oracle.linear_fwd(x[..., :128].reshape(-1, 128), w)) <= TOL


def _within_reference_tolerance(got, want, contraction):
    """The reference's own bound between its fused linear and bitsandbytes' (rtol = atol = 2e-3,
    solution/test_nf4.py:63-64). Its two sides multiply identical fp16 weights; here the weights
    inside the GEMM are rounded as fp16(table) * fp16(scale) and differ from the one-rounding
    decode by up to one fp16 step, an error that grows with the square root of the contraction
    length. Up to 1536 terms every element meets the bound; at 8960 terms 99.9 % do and none is
    further out than twice the bound."""
    err = (got.float() - want.float()).abs()
    allow = 2e-3 + 2e-3 * want.float().abs()
    if contraction <= 1536:
        assert bool((err <= allow).all()), float((err / allow).max())
    else:
        assert float((err <= allow).float().mean()) >= 0.999
        assert bool((err <= 2 * allow).all()), float((err / allow).max())


@pytest.mark.parametrize("n,k", [(8960, 1536), (1536, 8960), (1536, 1536)])
def test_training_shapes_at_2048_tokens_vs_oracle(cuda_lib, n, k):
    """gate/up, down and q/o of the 1.5B layer at the full 2048 tokens, forward and backward,
    every output element against the oracle: at the task's bound (max rel err <= 1e-2) and at the
    reference's elementwise 2e-3; the bias gradient equals the column sums of dy."""
    from hackaton_b200 import nf4_linear

    packed, state = synthetic_weight(n, k, True, seed=3 + n, device="cuda")
    w = oracle_weight(packed, state)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2048, k, generator=g).half()
    dy = torch.randn(2048, n, generator=g).half()
    bias = torch.zeros(n, device="cuda", dtype=torch.float16, requires_grad=True)
    xg = x.cuda().requires_grad_()
    y = nf4_linear(xg, packed, bias, state)
    y.backward(dy.cuda())
    y_ref, dx_ref = nf4_oracle.linear_fwd(x, w), nf4_oracle.linear_bwd(dy, w)
    assert rel(y, y_ref) <= TOL and rel(xg.grad, dx_ref) <= TOL
    _within_reference_tolerance(y.detach().cpu(), y_ref, k)
    _within_reference_tolerance(xg.grad.cpu(), dx_ref, n)
    torch.testing.assert_close(bias.grad.float().cpu(), dy.float().sum(0), rtol=2e-2, atol=2e-1)
    assert cuda_lib.device_status() == 0


def test_bad_arguments_raise(cuda_lib):
    from hackaton_b200 import nf4_linear

    packed, state = synthetic_weight(64, 128, True, seed=4, device="cuda")
    with pytest.raises(TypeError):
        nf4_linear(torch.randn(4, 128, device="cuda"), packed, None, state)  # fp32 input
    with pytest.raises(ValueError):
        nf4_linear(torch.randn(4, 64, device="cuda").half(), packed, None, state)  # wrong K
    packed2, state2 = synthetic_weight(64, 96, False, seed=4, device="cuda")  # K % 64 != 0
    with pytest.raises(cuda_lib.Nf4Error):
        nf4_linear(torch.randn(4, 96, device="cuda").half(), packed2, None, state2)


def test_split_k_equals_single_pass_and_is_deterministic(cuda_lib, monkeypatch):
    """Shapes with few output tiles split the K range over several CTAs through the fp32
    scratch; without scratch one CTA walks the whole range. Same numbers either way (up to fp32
    summation order), bit-identical from run to run, and the scratch needs no clearing between
    calls."""
    from hackaton_b200 import nf4 as nf4_mod

    n, k, m = 1536, 8960, 300      # down_proj: 2 x 6 tiles, 140 k-blocks
    packed, state = synthetic_weight(n, k, True, seed=8, device="cuda")
    need = cuda_lib.lib().nf4b200_workspace_bytes(n, k, m, 0)
    assert need > 0
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(m, k, generator=g, device="cuda").half()
    bias = torch.randn(n, generator=g, device="cuda").half()
    dy = torch.randn(m, n, generator=g, device="cuda").half()
    y1 = nf4_mod.linear_forward(x, packed, bias, state)
    y2 = nf4_mod.linear_forward(x, packed, bias, state)
    d1 = nf4_mod.linear_backward_dx(dy, packed, state)
    d2 = nf4_mod.linear_backward_dx(dy, packed, state)
    assert torch.equal(y1, y2) and torch.equal(d1, d2)
    monkeypatch.setattr(nf4_mod, "_workspace", lambda *a, **kw: (None, 0))
    y0 = nf4_mod.linear_forward(x, packed, bias, state)
    d0 = nf4_mod.linear_backward_dx(dy, packed, state)
    assert float((y1.float() - y0.float()).abs().max() / y0.float().abs().max()) < 2e-3
    assert float((d1.float() - d0.float()).abs().max() / d0.float().abs().max()) < 2e-3
    w = oracle_weight(packed, state)
    assert rel(y1, nf4_oracle.linear_fwd(x.cpu(), w, bias.cpu())) <= TOL
    cuda_lib.device_status()


def test_sm_limit_keeps_results(cuda_lib):
    """nf4b200_set_sm_limit: fewer SMs for the persistent grids, same numbers."""
    from hackaton_b200 import _lib
    from hackaton_b200.nf4 import linear_backward_dx, linear_forward

    packed, state = synthetic_weight(1536, 1536, True, seed=4, device="cuda")
    w = oracle_weight(packed, state)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(700, 1536, generator=g).half()
    dy = torch.randn(700, 1536, generator=g).half()
    try:
        _lib.set_sm_limit(64)
        y = linear_forward(x.cuda(), packed, None, state)
        dx = linear_backward_dx(dy.cuda(), packed, state)
    finally:
        _lib.set_sm_limit(0)
    assert rel(y, nf4_oracle.linear_fwd(x, w)) <= TOL
    assert rel(dx, nf4_oracle.linear_bwd(dy, w)) <= TOL
    cuda_lib.device_status()
