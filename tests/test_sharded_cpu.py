"""CPU, world_size 2 over gloo: the host logic of the column-sharded linear (shard ranges, the
all-gather of outputs and the all-reduce of input gradients). The CUDA kernels cannot run here,
so the two kernel wrappers are replaced, in this test only, by the oracle's arithmetic."""

import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hackaton_b200 import sharded
    from oracle import nf4_oracle
    from tests.util import oracle_weight

    sharded.linear_forward = lambda x, packed, bias, state: nf4_oracle.linear_fwd(
        x, oracle_weight(packed, state), bias)
    sharded.linear_backward_dx = lambda dy, packed, state: nf4_oracle.linear_bwd(
        dy, oracle_weight(packed, state))

    g = torch.Generator().manual_seed(0)
    n, k, m = 128, 64, 10
    w = (torch.randn(n, k, generator=g) * 0.02).half()
    x = torch.randn(m, k, generator=g).half()
    dy = torch.randn(m, n, generator=g).half()
    mod = sharded.ShardedNF4Linear.from_full_weight(w)
    lo, hi = sharded.shard_rows(n, world, rank)
    assert (lo, hi) == (rank * n // world, (rank + 1) * n // world)

    gathered, work = mod.forward(x, async_op=True)
    work.wait()
    y = sharded.ShardedNF4Linear.row_major(gathered)
    dx, work = mod.backward_dx(dy[:, lo:hi].contiguous(), async_op=True)
    work.wait()

    # expected: every rank's shard decoded separately, stacked along N
    shards = []
    for r in range(world):
        a, b = sharded.shard_rows(n, world, r)
        from hackaton_b200.quantize import quantize_nf4
        p, s = quantize_nf4(w[a:b].contiguous())
        shards.append(oracle_weight(p, s))
    w_all = torch.cat(shards, 0)
    ok_y = torch.allclose(y.float(), nf4_oracle.linear_fwd(x, w_all).float(), atol=2e-3, rtol=2e-3)
    ok_dx = torch.allclose(dx.float(), nf4_oracle.linear_bwd(dy, w_all).float(), atol=4e-3, rtol=4e-3)
    out[rank] = (bool(ok_y), bool(ok_dx), tuple(gathered.shape))
    dist.barrier()
    dist.destroy_process_group()


def test_column_sharded_linear_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        out = manager.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, out))
                 for port in [_free_port()] for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        for r in range(world):
            ok_y, ok_dx, shape = out[r]
            assert ok_y and ok_dx
            assert shape == (2, 10, 64)


def _paired_worker(rank, world, port, out):
    """gate/up output-sharded (no gather), SwiGLU on the shard, down input-sharded (one all-reduce);
    backward: down's dX shard stays local, gate/up's summed dX takes one all-reduce."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hackaton_b200 import group as group_mod
    from hackaton_b200 import sharded
    from hackaton_b200.quantize import quantize_nf4
    from oracle import nf4_oracle
    from tests.util import oracle_weight

    sharded.linear_forward = lambda x, packed, bias, state: nf4_oracle.linear_fwd(
        x, oracle_weight(packed, state), bias)
    sharded.linear_backward_dx = lambda dy, packed, state: nf4_oracle.linear_bwd(
        dy, oracle_weight(packed, state))
    group_mod.linear_forward_group = lambda x, ws: [nf4_oracle.linear_fwd(x, oracle_weight(p, s), None)
                                                    for p, s in ws]
    group_mod.linear_backward_dx_group = lambda gs, ws: sum(
        nf4_oracle.linear_bwd(g_, oracle_weight(p, s)).float() for g_, (p, s) in zip(gs, ws)).half()

    g = torch.Generator().manual_seed(0)
    hidden, inter, m = 64, 256, 10
    wg = (torch.randn(inter, hidden, generator=g) * 0.05).half()
    wu = (torch.randn(inter, hidden, generator=g) * 0.05).half()
    wd = (torch.randn(hidden, inter, generator=g) * 0.05).half()
    x = torch.randn(m, hidden, generator=g).half()
    dy = torch.randn(m, hidden, generator=g).half()
    gate = sharded.ShardedNF4Linear.from_full_weight(wg)
    up = sharded.ShardedNF4Linear.from_full_weight(wu)
    down = sharded.InputShardedNF4Linear.from_full_weight(wd)
    g_loc, u_loc = sharded.forward_local_group([gate, up], x)          # [m, inter / world] each
    h_loc = nf4_oracle.swiglu_fwd(g_loc, u_loc)
    y, work = down.forward(h_loc, async_op=True)
    work.wait()
    dh_loc, none = down.backward_dx(dy)
    d_gate, d_up = nf4_oracle.swiglu_bwd(dh_loc, g_loc, u_loc)
    dx, work = sharded.backward_dx_group([gate, up], [d_gate, d_up], async_op=True)
    work.wait()

    # expected: the same MLP on the full weights assembled from every rank's own shard
    def full(w, axis):
        parts = []
        for r in range(world):
            a, b = sharded.shard_rows(w.shape[axis], world, r)
            piece = w[a:b] if axis == 0 else w[:, a:b]
            parts.append(oracle_weight(*quantize_nf4(piece.contiguous())))
        return torch.cat(parts, axis)

    fg, fu, fd = full(wg, 0), full(wu, 0), full(wd, 1)
    gate_f, up_f = nf4_oracle.linear_fwd(x, fg), nf4_oracle.linear_fwd(x, fu)
    y_ref = nf4_oracle.linear_fwd(nf4_oracle.swiglu_fwd(gate_f, up_f), fd)
    dg_f, du_f = nf4_oracle.swiglu_bwd(nf4_oracle.linear_bwd(dy, fd), gate_f, up_f)
    dx_ref = dg_f.float() @ fg.float() + du_f.float() @ fu.float()
    out[rank] = (nf4_oracle.max_rel_err(y, y_ref), nf4_oracle.max_rel_err(dx, dx_ref), none is None,
                 tuple(g_loc.shape), tuple(dh_loc.shape))
    dist.barrier()
    dist.destroy_process_group()


def test_paired_sharding_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        out = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_paired_worker, args=(r, world, port, out)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        for r in range(world):
            err_y, err_dx, no_work, g_shape, dh_shape = out[r]
            assert err_y <= 1e-2 and err_dx <= 1e-2 and no_work
            assert g_shape == (10, 128) and dh_shape == (10, 128)


def test_input_shards_must_be_whole_blocks():
    import pytest

    from hackaton_b200.quantize import quantize_nf4
    from hackaton_b200.sharded import InputShardedNF4Linear

    packed, state = quantize_nf4((torch.randn(16, 96) * 0.02).half())
    with pytest.raises(ValueError):
        InputShardedNF4Linear(packed, state, 96)      # 96 columns: not a multiple of 64


def test_uneven_split_is_rejected():
    import pytest

    from hackaton_b200.sharded import shard_rows

    with pytest.raises(ValueError):
        shard_rows(100, 8, 0)
