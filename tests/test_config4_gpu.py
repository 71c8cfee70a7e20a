"""GPU: the 7B-shaped projections (hidden 3584, intermediate 18944, k/v 512) at 8192 tokens, whole
and as the shards a 2-, 4- and 8-GPU run launches, against the CPU oracle.

The multi-GPU layouts only ever launch the single-GPU kernels on a shard of a weight, so every
shard shape is checked here on one GPU: the shards of one weight run one after the other through
the same grouped calls the sharded modules make, their outputs are concatenated (output shards)
or summed (input shards, the arithmetic an all-reduce performs) and compared with the oracle on
the weight assembled from the shards. The oracle sees a slice of the token rows (the first 192
and the last 64 of 8192: both ends of the row range, first and last row tile); the kernels run
all 8192.
"""

from types import SimpleNamespace

import pytest
import torch

from oracle import nf4_oracle
from tests.util import oracle_weight

pytestmark = pytest.mark.gpu
TOL = 1e-2
M = 8192
HIDDEN, INTER, KV = 3584, 18944, 512


def _rows():
    return torch.cat((torch.arange(0, 192), torch.arange(M - 64, M)))


def _weight(n, k, seed):
    from hackaton_b200.quantize import quantize_nf4

    g = torch.Generator(device="cuda").manual_seed(seed)
    w = (torch.randn(n, k, generator=g, device="cuda") * 0.02).half()
    packed, state = quantize_nf4(w, blocksize=64, compress_statistics=True)
    return packed.reshape(-1), state


def _act(cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(M, cols, generator=g, device="cuda").half()


def _mod(packed, state):
    return SimpleNamespace(packed=packed, state=state, world=1, group=None)


def _rel(got_rows, want):
    return nf4_oracle.max_rel_err(got_rows, want)


@pytest.mark.parametrize("name,n,k", [("q", HIDDEN, HIDDEN), ("k", KV, HIDDEN),
                                      ("gate", INTER, HIDDEN), ("down", HIDDEN, INTER)])
def test_full_7b_projection_at_8192_tokens(cuda_lib, name, n, k):
    from hackaton_b200.nf4 import linear_backward_dx, linear_forward

    packed, state = _weight(n, k, seed=n + k)
    w = oracle_weight(packed, state)
    x, dy = _act(k, 1), _act(n, 2)
    y = linear_forward(x, packed, None, state)
    dx = linear_backward_dx(dy, packed, state)
    rows = _rows()
    assert _rel(y[rows.cuda()].cpu(), nf4_oracle.linear_fwd(x[rows.cuda()].cpu(), w)) <= TOL
    assert _rel(dx[rows.cuda()].cpu(), nf4_oracle.linear_bwd(dy[rows.cuda()].cpu(), w)) <= TOL
    assert cuda_lib.device_status() == 0


def _output_sharded_group(cuda_lib, widths, world, seed):
    """q/k/v or gate/up split along their output features: every rank's grouped forward (outputs
    kept as shards) and grouped backward (dX summed over the group on the rank, then over the
    ranks)."""
    from hackaton_b200.sharded import backward_dx_group, forward_local_group

    rows = _rows()
    rows_dev = rows.cuda()
    x = _act(HIDDEN, seed)
    x_cpu = x[rows_dev].cpu()
    dx_sum = torch.zeros(M, HIDDEN, dtype=torch.float32, device="cuda")
    dx_ref = torch.zeros(len(rows), HIDDEN, dtype=torch.float32)
    for rank in range(world):
        shards = [_weight(n // world, HIDDEN, seed * 100 + rank * 10 + i) for i, n in enumerate(widths)]
        mods = [_mod(p, s) for p, s in shards]
        ws = [oracle_weight(p, s) for p, s in shards]
        outs = forward_local_group(mods, x)
        for y, w, n in zip(outs, ws, widths):
            assert y.shape == (M, n // world)
            assert _rel(y[rows_dev].cpu(), nf4_oracle.linear_fwd(x_cpu, w)) <= TOL, (world, rank, n)
        dys = [_act(n // world, seed + 7 + rank * 3 + i) for i, n in enumerate(widths)]
        dx, work = backward_dx_group(mods, dys)
        assert work is None
        dx_sum += dx.float()
        for dy, w in zip(dys, ws):
            dx_ref += dy[rows_dev].cpu().float() @ w.float()
    assert _rel(dx_sum[rows_dev].cpu(), dx_ref) <= TOL, world
    assert cuda_lib.device_status() == 0


def _input_sharded(cuda_lib, n, k_total, world, seed):
    """o or down split along their input features: forward = local GEMM on the rank's input shard,
    outputs summed over the ranks; backward = the rank's own shard of dX, no exchange."""
    from hackaton_b200.sharded import InputShardedNF4Linear

    rows = _rows()
    rows_dev = rows.cuda()
    dy = _act(n, seed + 1)
    dy_cpu = dy[rows_dev].cpu()
    y_sum = torch.zeros(M, n, dtype=torch.float32, device="cuda")
    y_ref = torch.zeros(len(rows), n, dtype=torch.float32)
    for rank in range(world):
        packed, state = _weight(n, k_total // world, seed * 100 + rank)
        mod = InputShardedNF4Linear(packed, state, k_total // world)   # one process: world of 1
        w = oracle_weight(packed, state)
        x = _act(k_total // world, seed + 2 + rank)
        y, work = mod.forward(x)
        assert work is None
        y_sum += y.float()                     # fp16 partial sums, as the all-reduce receives them
        y_ref += x[rows_dev].cpu().float() @ w.float().t()
        dx, _ = mod.backward_dx(dy)
        assert dx.shape == (M, k_total // world)
        assert _rel(dx[rows_dev].cpu(), nf4_oracle.linear_bwd(dy_cpu, w)) <= TOL, (world, rank)
    assert _rel(y_sum[rows_dev].cpu(), y_ref) <= TOL, world
    assert cuda_lib.device_status() == 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_qkv_shards(cuda_lib, world):
    """q 3584/G rows, k and v 512/G rows (64 at G = 8), one grouped launch per rank."""
    _output_sharded_group(cuda_lib, (HIDDEN, KV, KV), world, seed=3)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gate_up_shards(cuda_lib, world):
    """gate and up 18944/G rows each (2368 at G = 8: not a multiple of the 256-wide tile)."""
    _output_sharded_group(cuda_lib, (INTER, INTER), world, seed=5)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_o_proj_input_shards(cuda_lib, world):
    """o: 3584 x (3584/G) per rank (448 columns at G = 8)."""
    _input_sharded(cuda_lib, HIDDEN, HIDDEN, world, seed=11)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_down_proj_input_shards(cuda_lib, world):
    """down: 3584 x (18944/G) per rank (2368 columns at G = 8)."""
    _input_sharded(cuda_lib, HIDDEN, INTER, world, seed=13)


@pytest.mark.parametrize("world", [2, 8])
def test_gathered_layout_shards(cuda_lib, world):
    """The all-gather layout: every projection split along its output features, also o and down
    (o 3584/G x 3584, down 3584/G x 18944): forward shard and the rank's partial dX."""
    from hackaton_b200.nf4 import linear_backward_dx, linear_forward

    rows_dev = _rows().cuda()
    for n, k, seed in ((HIDDEN, HIDDEN, 17), (HIDDEN, INTER, 19)):
        x, dy = _act(k, seed), _act(n // world, seed + 1)
        for rank in (0, world - 1):
            packed, state = _weight(n // world, k, seed * 10 + rank)
            w = oracle_weight(packed, state)
            y = linear_forward(x, packed, None, state)
            dx = linear_backward_dx(dy, packed, state)
            assert _rel(y[rows_dev].cpu(), nf4_oracle.linear_fwd(x[rows_dev].cpu(), w)) <= TOL
            assert _rel(dx[rows_dev].cpu(), nf4_oracle.linear_bwd(dy[rows_dev].cpu(), w)) <= TOL
    assert cuda_lib.device_status() == 0


@pytest.mark.parametrize("world", [2, 8])
def test_qkv_shards_with_lora(cuda_lib, world):
    """LoRA on the sharded q and v (A replicated, B split with W): one rank's grouped forward,
    grouped dX with both rank-16 shares, and the factors' gradients, at the shard shapes of 2 and
    8 GPUs (v: 256 and 64 rows), against the oracle. 2048 token rows keep the CPU side short."""
    from hackaton_b200.sharded import ShardedNF4Linear, backward_dx_group, forward_local_group, lora_weight_grads

    m, scaling = 2048, 2.0
    g = torch.Generator(device="cuda").manual_seed(40 + world)
    x = torch.randn(m, HIDDEN, generator=g, device="cuda").half()
    mods, refs, grads = [], [], []
    for i, n in enumerate((HIDDEN // world, KV // world, KV // world)):
        packed, state = _weight(n, HIDDEN, 400 + world * 10 + i)
        a = b = None
        if i != 1:
            a = ((torch.rand(16, HIDDEN, generator=g, device="cuda") * 2 - 1) / HIDDEN ** 0.5).half()
            b = (torch.randn(n, 16, generator=g, device="cuda") * 0.05).half()
        mods.append(ShardedNF4Linear(packed, state, n, lora_a=a, lora_b=b, scaling=scaling))
        refs.append((oracle_weight(packed, state), a, b))
        grads.append(torch.randn(m, n, generator=g, device="cuda").half())
    ys, xas = forward_local_group(mods, x, return_lora_inputs=True)
    dx, work, us = backward_dx_group(mods, grads, return_lora_inputs=True)
    wgrads, works = lora_weight_grads(mods, x, grads, xas, us)
    assert work is None and works == [] and sorted(wgrads) == [0, 2]
    x_cpu = x.cpu()
    dx_ref = torch.zeros(m, HIDDEN)
    for i, (y, (w, a, b), dy) in enumerate(zip(ys, refs, grads)):
        if a is None:
            assert _rel(y.cpu(), nf4_oracle.linear_fwd(x_cpu, w)) <= TOL
            dx_ref += nf4_oracle.linear_bwd(dy.cpu(), w).float()
            continue
        y_ref, _ = nf4_oracle.lora_fwd(x_cpu, w, a.cpu(), b.cpu(), scaling)
        d_ref, da_ref, db_ref = nf4_oracle.lora_bwd(dy.cpu(), x_cpu, w, a.cpu(), b.cpu(), scaling)
        dx_ref += d_ref.float()
        assert _rel(y.cpu(), y_ref) <= TOL
        assert _rel(wgrads[i][0].cpu(), da_ref) <= TOL
        assert _rel(wgrads[i][1].cpu(), db_ref) <= TOL
    assert _rel(dx.cpu(), dx_ref) <= TOL
    assert cuda_lib.device_status() == 0
