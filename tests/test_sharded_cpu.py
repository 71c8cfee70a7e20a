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


def test_uneven_split_is_rejected():
    import pytest

    from hackaton_b200.sharded import shard_rows

    with pytest.raises(ValueError):
        shard_rows(100, 8, 0)
