"""GPU: the weight-streaming forward kernel that serves M <= 64 (decode-like token counts,
M in {1, 4, 16, 64}) against the oracle, with bias and the LoRA term, and
against the tensor-core kernel it replaces at these sizes."""

import pytest
import torch

from oracle import nf4_oracle
from tests.util import oracle_weight, synthetic_weight

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.mark.parametrize("m", [1, 4, 5, 16, 33, 64])
@pytest.mark.parametrize("n,k", [(1536, 1536), (256, 1536), (1536, 8960), (8960, 1536), (48, 64)])
def test_small_m_forward_vs_oracle(cuda_lib, m, n, k):
    from hackaton_b200.nf4 import linear_forward

    packed, state = synthetic_weight(n, k, True, seed=n + m, device="cuda")
    w = oracle_weight(packed, state)
    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, k, generator=g).half()
    bias = torch.randn(n, generator=g).half()
    y = linear_forward(x.cuda(), packed, bias.cuda(), state)
    assert nf4_oracle.max_rel_err(y.cpu(), nf4_oracle.linear_fwd(x, w, bias)) <= TOL
    cuda_lib.device_status()


@pytest.mark.parametrize("m", [1, 16, 64])
def test_small_m_lora_term(cuda_lib, m):
    from hackaton_b200 import nf4_lora_linear

    n, k = 1536, 1536
    packed, state = synthetic_weight(n, k, True, seed=7, device="cuda")
    w = oracle_weight(packed, state)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(m, k, generator=g).half()
    a = ((torch.rand(16, k, generator=g) * 2 - 1) / k ** 0.5).half()
    b = (torch.randn(n, 16, generator=g) * 0.2).half()
    y = nf4_lora_linear(x.cuda(), packed, None, state, a.cuda(), b.cuda(), 2.0)
    y_ref, _ = nf4_oracle.lora_fwd(x, w, a, b, 2.0)
    assert nf4_oracle.max_rel_err(y.cpu(), y_ref) <= TOL
    assert nf4_oracle.max_rel_err(nf4_oracle.linear_fwd(x, w), y_ref) > 5 * TOL  # term is visible


def test_small_m_matches_tensor_core_kernel(cuda_lib):
    """Same weight, M = 16: the streaming kernel (scale table present) and the tcgen05 kernel
    (no table, so the call is not eligible for the streaming kernel) agree to fp16 rounding."""
    from hackaton_b200 import nf4

    n, k, m = 1536, 1536, 16
    x = torch.randn(m, k, device="cuda").half()
    outs = []
    for prepared in (True, False):
        nf4.PREPARED_SCALES = prepared
        try:
            packed, state = synthetic_weight(n, k, True, seed=5, device="cuda")
            outs.append(nf4.linear_forward(x, packed, None, state).float())
        finally:
            nf4.PREPARED_SCALES = True
    assert (outs[0] - outs[1]).abs().max() <= 2e-3 * outs[1].abs().max()


def test_fresh_weights_first_calls_vs_reference(cuda_lib):
    """First calls on freshly created weights (cold caches, scale table just built), M <= 128 with
    split-K, several weights in a row: each of two calls in a row is compared with the fp32
    product of the bit-exact standalone decode (itself pinned to the oracle), the first weight of
    every token count also with the CPU oracle, and the two calls must give the same bits."""
    from hackaton_b200.nf4 import dequantize_nf4, linear_forward

    n, k = 1536, 8960
    for rep in range(6):
        for m in (33, 64, 20, 128):
            packed, state = synthetic_weight(n, k, True, seed=100 + rep * 7 + m, device="cuda")
            x = torch.randn(m, k, device="cuda").half()
            y1 = linear_forward(x, packed, None, state)
            y2 = linear_forward(x, packed, None, state)
            w_dev = dequantize_nf4(packed, state)
            want = x.float() @ w_dev.float().t()
            scale = float(want.abs().max())
            for call, y in enumerate((y1, y2)):
                err = float((y.float() - want).abs().max()) / scale
                assert err <= 2e-3, (rep, m, call, err)
            assert torch.equal(y1, y2), (rep, m)
            if rep == 0:
                w = oracle_weight(packed, state)
                assert torch.equal(w_dev.cpu(), w)
                assert nf4_oracle.max_rel_err(y1.cpu(), nf4_oracle.linear_fwd(x.cpu(), w)) <= TOL
    assert cuda_lib.device_status() == 0


@pytest.mark.parametrize("nested", [True, False])
def test_code_ring_hand_back_under_load(cuda_lib, nested):
    """The code ring of the fused kernel is read with ordinary shared-memory loads and re-filled by
    TMA; the hand-back between the two has to order them (a proxy fence). When it did not, a warp
    could decode part of its rows from the next k-block's codes: a few wrong output columns in
    about half of the calls at these shapes. Fresh weights, both scale paths, token counts of
    every kernel variant, forward and backward, each call against the fp32 product of the
    standalone decode (bit-equal to the oracle, which the first weight re-checks)."""
    import copy

    from hackaton_b200 import nf4

    for i in range(10):
        n, k = ((1536, 8960), (1536, 8960), (8960, 1536), (1536, 1536))[i % 4]
        packed, state = synthetic_weight(n, k, nested, seed=900 + i, device="cuda")
        bare = copy.copy(state)            # same tensors, no cached descriptor, no scale table
        w = nf4.dequantize_nf4(packed, state)
        if i == 0:
            assert torch.equal(w.cpu(), oracle_weight(packed, state))
        wf = w.float()
        for m in (1, 20, 33, 64, 128, 300, 2048):
            x = torch.randn(m, k, device="cuda").half()
            dy = torch.randn(m, n, device="cuda").half()
            want_y, want_dx = x.float() @ wf.t(), dy.float() @ wf
            try:
                for prepared, st in ((True, state), (False, bare)):
                    nf4.PREPARED_SCALES = prepared
                    for call in range(2):
                        y = nf4.linear_forward(x, packed, None, st)
                        dx = nf4.linear_backward_dx(dy, packed, st)
                        ey = float((y.float() - want_y).abs().max() / want_y.abs().max())
                        edx = float((dx.float() - want_dx).abs().max() / want_dx.abs().max())
                        assert ey <= 2e-3 and edx <= 2e-3, (i, n, k, m, prepared, call, ey, edx)
            finally:
                nf4.PREPARED_SCALES = True
    assert cuda_lib.device_status() == 0


@pytest.mark.parametrize("m", [1, 4, 5, 16])
@pytest.mark.parametrize("n,k", [(1536, 1536), (256, 1536), (1536, 8960), (8960, 1536), (48, 64)])
def test_small_m_backward_vs_oracle(cuda_lib, m, n, k):
    """dX = dY . W for up to 16 token rows: the weight-streaming backward kernel (row slabs summed
    as fp32 planes) against the oracle, twice (the scratch needs no clearing between calls)."""
    from hackaton_b200.nf4 import linear_backward_dx

    packed, state = synthetic_weight(n, k, True, seed=n + 3 * m, device="cuda")
    w = oracle_weight(packed, state)
    g = torch.Generator().manual_seed(m)
    dy = torch.randn(m, n, generator=g).half()
    want = nf4_oracle.linear_bwd(dy, w)
    for _ in range(2):
        dx = linear_backward_dx(dy.cuda(), packed, state)
        assert nf4_oracle.max_rel_err(dx.cpu(), want) <= TOL
    assert cuda_lib.device_status() == 0


@pytest.mark.parametrize("m", [1, 7, 16, 40])
def test_small_m_group_with_lora(cuda_lib, m):
    """q/k/v sharing one input at decode-like token counts: one streaming launch forward (three
    outputs, LoRA on q and v), one backward (summed dX with both LoRA shares), through autograd."""
    from hackaton_b200 import Projection, nf4_linear_group

    k = 1536
    g = torch.Generator().manual_seed(11 + m)
    x = torch.randn(m, k, generator=g).half()
    projs, refs, grads = [], [], []
    for i, n in enumerate((1536, 256, 256)):
        packed, state = synthetic_weight(n, k, True, seed=50 + i, device="cuda")
        w = oracle_weight(packed, state)
        a = b = None
        if i != 1:
            a = ((torch.rand(16, k, generator=g) * 2 - 1) / k ** 0.5).half()
            b = (torch.randn(n, 16, generator=g) * 0.1).half()
        projs.append(Projection(packed, state, None, None if a is None else a.cuda().requires_grad_(),
                                None if b is None else b.cuda().requires_grad_(), 2.0))
        refs.append((w, a, b))
        grads.append(torch.randn(m, n, generator=g).half())
    xg = x.cuda().requires_grad_()
    ys = nf4_linear_group(xg, projs)
    torch.autograd.backward(list(ys), [d.cuda() for d in grads])
    dx_ref = torch.zeros(m, k)
    for y, (w, a, b), dy in zip(ys, refs, grads):
        if a is None:
            want = nf4_oracle.linear_fwd(x, w)
            dx_ref += nf4_oracle.linear_bwd(dy, w).float()
        else:
            want, _ = nf4_oracle.lora_fwd(x, w, a, b, 2.0)
            dx_ref += nf4_oracle.lora_bwd(dy, x, w, a, b, 2.0)[0].float()
        assert nf4_oracle.max_rel_err(y.detach().cpu(), want) <= TOL
    assert nf4_oracle.max_rel_err(xg.grad.cpu(), dx_ref) <= TOL
    assert cuda_lib.device_status() == 0
