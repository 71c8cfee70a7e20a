"""GPU: problems that run as 512-row x 128-column tiles in a single wave (few output columns, more
than 256 token rows, a scale table per weight: q/k/v and o at 2048 tokens) against the CPU oracle:
ragged edges in every direction, bias, the rank-16 term, groups in both directions.

The oracle's fp32 product is the reference; the tile shape changes which CTA adds what, never the
order in which the k-blocks of one output element are added, so the whole-contraction shapes are
also compared bit for bit with the same call on the weight without a table (which cannot take
these tiles and runs as 256-column tiles)."""

import pytest
import torch

from oracle import nf4_oracle
from tests.util import oracle_weight, synthetic_weight

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _inputs(m, n, k, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(m, k, generator=g, device="cuda").half()
    dy = torch.randn(m, n, generator=g, device="cuda").half()
    return x, dy


# (m, n, k): full tiles; rows and columns that end inside a tile (n % 128 = 8: the second CTA of the
# last pair has no weight rows at all); a single 64-deep k-block; the longest contraction taken
@pytest.mark.parametrize("m,n,k", [(2048, 1536, 1536), (700, 392, 640), (513, 136, 64),
                                   (1024, 256, 2560), (2048, 520, 1536)])
def test_forward_and_backward_vs_oracle(cuda_lib, m, n, k):
    from hackaton_b200.nf4 import linear_backward_dx, linear_forward

    packed, state = synthetic_weight(n, k, True, seed=m + n + k, device="cuda")
    w = oracle_weight(packed, state)
    x, dy = _inputs(m, n, k, seed=k)
    bias = (torch.arange(n, device="cuda") % 7 - 3).half() * 0.25
    y = linear_forward(x, packed, bias, state)
    dx = linear_backward_dx(dy, packed, state)
    y_ref = nf4_oracle.linear_fwd(x.cpu(), w).float() + bias.cpu().float()
    assert nf4_oracle.max_rel_err(y.cpu(), y_ref) <= TOL
    assert nf4_oracle.max_rel_err(dx.cpu(), nf4_oracle.linear_bwd(dy.cpu(), w)) <= TOL
    assert cuda_lib.device_status() == 0


def test_same_bits_as_the_wide_tiles(cuda_lib):
    """2048 x 1536 x 1536: with a table the call runs as 128-wide tiles, without one as 256-wide
    tiles, neither with K-slices: every output element is the same sum in the same order."""
    from hackaton_b200 import nf4

    m, n, k = 2048, 1536, 1536
    x, dy = _inputs(m, n, k, seed=4)
    out = {}
    try:
        for prepared in (True, False):
            nf4.PREPARED_SCALES = prepared
            packed, state = synthetic_weight(n, k, True, seed=6, device="cuda")
            out[prepared] = (nf4.linear_forward(x, packed, None, state),
                             nf4.linear_backward_dx(dy, packed, state))
    finally:
        nf4.PREPARED_SCALES = True
    assert torch.equal(out[True][0], out[False][0])
    assert torch.equal(out[True][1], out[False][1])
    assert cuda_lib.device_status() == 0


@pytest.mark.parametrize("m,n,k", [(2048, 1536, 1536), (600, 200, 320)])
def test_rank16_term(cuda_lib, m, n, k):
    from hackaton_b200 import nf4_lora_linear

    packed, state = synthetic_weight(n, k, True, seed=m + n, device="cuda")
    w = oracle_weight(packed, state)
    x, dy = _inputs(m, n, k, seed=m)
    g = torch.Generator(device="cuda").manual_seed(n)
    a = ((torch.rand(16, k, generator=g, device="cuda") * 2 - 1) / k ** 0.5).half()
    b = (torch.randn(n, 16, generator=g, device="cuda") * 0.2).half()
    scaling = 2.0
    xg, ag, bg = x.clone().requires_grad_(), a.clone().requires_grad_(), b.clone().requires_grad_()
    y = nf4_lora_linear(xg, packed, None, state, ag, bg, scaling)
    y.backward(dy)
    torch.cuda.synchronize()
    y_ref, _ = nf4_oracle.lora_fwd(x.cpu(), w, a.cpu(), b.cpu(), scaling)
    dx_ref, da_ref, db_ref = nf4_oracle.lora_bwd(dy.cpu(), x.cpu(), w, a.cpu(), b.cpu(), scaling)
    assert nf4_oracle.max_rel_err(y.cpu(), y_ref) <= TOL
    assert nf4_oracle.max_rel_err(xg.grad.cpu(), dx_ref) <= TOL
    assert nf4_oracle.max_rel_err(ag.grad.cpu(), da_ref) <= TOL
    assert nf4_oracle.max_rel_err(bg.grad.cpu(), db_ref) <= TOL
    assert nf4_oracle.max_rel_err(nf4_oracle.linear_fwd(x.cpu(), w), y_ref) > 5 * TOL
    assert cuda_lib.device_status() == 0


@pytest.mark.parametrize("m,widths,k", [(2048, (1536, 256, 256), 1536), (900, (392, 72, 136), 448)])
def test_groups_in_both_directions(cuda_lib, m, widths, k):
    """q/k/v-like groups: the forward stacks the members' 128-wide tiles into one unit list, the
    backward chains their k-blocks into one contraction (32 k-blocks for 1536 + 256 + 256)."""
    from hackaton_b200.group import linear_backward_dx_group, linear_forward_group

    weights = [synthetic_weight(n, k, True, seed=10 * i + n, device="cuda") for i, n in enumerate(widths)]
    ws = [oracle_weight(p, s) for p, s in weights]
    g = torch.Generator(device="cuda").manual_seed(m)
    x = torch.randn(m, k, generator=g, device="cuda").half()
    dys = [torch.randn(m, n, generator=g, device="cuda").half() for n in widths]
    ys = linear_forward_group(x, weights)
    dx = linear_backward_dx_group(dys, weights)
    for y, w in zip(ys, ws):
        assert nf4_oracle.max_rel_err(y.cpu(), nf4_oracle.linear_fwd(x.cpu(), w)) <= TOL
    dx_ref = sum(dy.cpu().float() @ w.float() for dy, w in zip(dys, ws))
    assert nf4_oracle.max_rel_err(dx.cpu(), dx_ref) <= TOL
    assert cuda_lib.device_status() == 0
