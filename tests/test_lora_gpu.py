"""GPU: LoRA r=16 fused into the NF4 linear (forward, dX, dA, dB) against the oracle formula.
Parity unpinned: the reference has no LoRA test (peft's code is third-party)."""

import pytest
import torch

from oracle import nf4_oracle
from tests.util import oracle_weight, synthetic_weight

pytestmark = pytest.mark.gpu
TOL = 1e-2


def make(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).half()
    dy = torch.randn(m, n, generator=g).half()
    a = ((torch.rand(16, k, generator=g) * 2 - 1) / k ** 0.5).half()   # U(+-1/sqrt(K))
    b = (torch.randn(n, 16, generator=g) * 0.01).half()                # N(0, 0.01)
    return x, dy, a, b


@pytest.mark.parametrize("m,n,k", [(2048, 1536, 1536), (300, 256, 1536), (77, 264, 192),
                                   (1, 256, 64), (128, 512, 128)])
def test_lora_forward_backward_vs_oracle(cuda_lib, m, n, k):
    from hackaton_b200 import nf4_lora_linear

    packed, state = synthetic_weight(n, k, True, seed=m + n, device="cuda")
    w = oracle_weight(packed, state)
    x, dy, a, b = make(m, n, k, seed=m)
    # make the low-rank term visible next to the base product
    b = b * 20
    scaling = 2.0
    xg = x.cuda().requires_grad_()
    ag = a.cuda().requires_grad_()
    bg = b.cuda().requires_grad_()
    y = nf4_lora_linear(xg, packed, None, state, ag, bg, scaling)
    y.backward(dy.cuda())
    torch.cuda.synchronize()
    y_ref, _ = nf4_oracle.lora_fwd(x, w, a, b, scaling)
    dx_ref, da_ref, db_ref = nf4_oracle.lora_bwd(dy, x, w, a, b, scaling)
    assert nf4_oracle.max_rel_err(y.cpu(), y_ref) <= TOL
    assert nf4_oracle.max_rel_err(xg.grad.cpu(), dx_ref) <= TOL
    assert nf4_oracle.max_rel_err(ag.grad.cpu(), da_ref) <= TOL
    assert nf4_oracle.max_rel_err(bg.grad.cpu(), db_ref) <= TOL
    # the low-rank term really is in there
    base = nf4_oracle.linear_fwd(x, w)
    assert nf4_oracle.max_rel_err(base, y_ref) > 5 * TOL
    cuda_lib.device_status()


def test_lora_with_dropout_branch(cuda_lib):
    """x_lora != x (peft's lora_dropout in training): the two input gradients stay separate."""
    from hackaton_b200 import nf4_lora_linear

    m, n, k = 200, 256, 128
    packed, state = synthetic_weight(n, k, True, seed=1, device="cuda")
    w = oracle_weight(packed, state)
    x, dy, a, b = make(m, n, k, seed=3)
    b = b * 20
    g = torch.Generator().manual_seed(5)
    mask = (torch.rand(m, k, generator=g) > 0.05).half() / 0.95
    xl = (x * mask).half()
    xg, xlg = x.cuda().requires_grad_(), xl.cuda().requires_grad_()
    y = nf4_lora_linear(xg, packed, None, state, a.cuda(), b.cuda(), 2.0, x_lora=xlg)
    y.backward(dy.cuda())
    y_ref = (x.float() @ w.float().t() + 2.0 * (xl.float() @ a.float().t()) @ b.float().t())
    assert nf4_oracle.max_rel_err(y.cpu(), y_ref) <= TOL
    assert nf4_oracle.max_rel_err(xg.grad.cpu(), dy.float() @ w.float()) <= TOL
    dxl_ref = 2.0 * (dy.float() @ b.float()) @ a.float()
    assert nf4_oracle.max_rel_err(xlg.grad.cpu(), dxl_ref) <= TOL


def test_batched_lora_kernels_match_single(cuda_lib):
    """nf4b200_lora_down_batch / _grad_batch: same results as one call per problem."""
    from hackaton_b200.lora import lora_down, lora_down_batch, lora_grad, lora_grad_batch

    torch.manual_seed(11)
    m = 777
    x = torch.randn(m, 1536, device="cuda").half()
    a_q = (torch.randn(16, 1536, device="cuda") * 0.05).half()
    a_v = (torch.randn(16, 1536, device="cuda") * 0.05).half()
    got = lora_down_batch([x, x], [a_q, a_v], True, [2.0, 0.5])
    want = [lora_down(x, a_q, True, 2.0), lora_down(x, a_v, True, 0.5)]
    for g, w in zip(got, want):
        assert torch.equal(g, w)

    dy_q = torch.randn(m, 1536, device="cuda").half()
    dy_v = torch.randn(m, 256, device="cuda").half()
    b_q = (torch.randn(1536, 16, device="cuda") * 0.05).half()
    b_v = (torch.randn(256, 16, device="cuda") * 0.05).half()
    got = lora_down_batch([dy_q, dy_v], [b_q, b_v], False, [2.0, 2.0])
    want = [lora_down(dy_q, b_q, False, 2.0), lora_down(dy_v, b_v, False, 2.0)]
    for g, w in zip(got, want):
        assert torch.equal(g, w)

    u_q, u_v = want
    xa_q, xa_v = lora_down(x, a_q, True, 2.0), lora_down(x, a_v, True, 2.0)
    got = lora_grad_batch([x, dy_q, x, dy_v], [u_q, xa_q, u_v, xa_v], [True, False, True, False])
    want = [lora_grad(x, u_q, True), lora_grad(dy_q, xa_q, False), lora_grad(x, u_v, True),
            lora_grad(dy_v, xa_v, False)]
    for g, w in zip(got, want):
        assert g.shape == w.shape
        # fp32 atomics: the order of the block sums is not fixed
        assert (g - w).abs().max() <= 1e-4 * w.abs().max().clamp_min(1.0)
