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
    group_mod.linear_forward_group = lambda x, ws, *lora: [
        nf4_oracle.linear_fwd(x, oracle_weight(p, s), None) for p, s in ws]
    group_mod.linear_backward_dx_group = lambda gs, ws, *lora: sum(
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


def test_slices_of_a_quantised_weight_decode_to_slices_of_its_decode():
    """`slice_rows` / `slice_cols`: a shard cut out of an already quantised (double-quantised)
    weight decodes to exactly the matching rows / columns of the full weight's decode."""
    from hackaton_b200.quantize import quantize_nf4
    from hackaton_b200.sharded import slice_cols, slice_rows
    from tests.util import oracle_weight

    g = torch.Generator().manual_seed(3)
    for nested in (True, False):
        w = (torch.randn(96, 448, generator=g) * 0.02).half()      # 448 = 7 blocks of 64 per row
        packed, state = quantize_nf4(w, compress_statistics=nested)
        full = oracle_weight(packed, state)
        for lo, hi in ((0, 12), (12, 24), (84, 96), (5, 77)):
            p, s = slice_rows(packed, state, lo, hi)
            assert torch.equal(oracle_weight(p, s), full[lo:hi])
        for lo, hi in ((0, 64), (64, 448), (128, 192)):
            p, s = slice_cols(packed, state, lo, hi)
            assert torch.equal(oracle_weight(p, s), full[:, lo:hi])
    import pytest
    with pytest.raises(ValueError):
        slice_cols(packed, state, 32, 96)        # not on a block boundary


def _lora_worker(rank, world, port, out):
    """q and v output-sharded with LoRA (A replicated, B split by rows), k without: forward shards,
    the all-reduced dX with its LoRA share, dA all-reduced over ranks, dB local."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hackaton_b200 import group as group_mod
    from hackaton_b200 import lora as lora_mod
    from hackaton_b200 import sharded
    from hackaton_b200.quantize import quantize_nf4
    from oracle import nf4_oracle
    from tests.util import oracle_weight

    def fwd_group(x, ws, biases=None, xas=None, lora_bs=None):
        ys = []
        for i, (p, s) in enumerate(ws):
            y = x.float() @ oracle_weight(p, s).float().t()
            if xas is not None and xas[i] is not None:
                y = y + xas[i].float() @ lora_bs[i].float().t()
            ys.append(y.half())
        return ys

    def bwd_group(gs, ws, us=None, lora_as=None):
        dx = 0
        for i, (g_, (p, s)) in enumerate(zip(gs, ws)):
            dx = dx + g_.float() @ oracle_weight(p, s).float()
            if us is not None and us[i] is not None:
                dx = dx + us[i].float() @ lora_as[i].float()
        return dx.half()

    group_mod.linear_forward_group, group_mod.linear_backward_dx_group = fwd_group, bwd_group
    lora_mod.lora_down_batch = lambda inputs, ps, rank_major, scalings: [
        (sc * (i_.float() @ (p_.float().t() if rank_major else p_.float()))).half()
        for i_, p_, sc in zip(inputs, ps, scalings)]
    lora_mod.lora_grad_batch = lambda zs, ss, rms: [
        (s_.float().t() @ z_.float()) if rm else (z_.float().t() @ s_.float())
        for z_, s_, rm in zip(zs, ss, rms)]

    g = torch.Generator().manual_seed(0)
    k, nq, nk, m, scaling = 128, 64, 32, 12, 2.0
    wq = (torch.randn(nq, k, generator=g) * 0.05).half()
    wk = (torch.randn(nk, k, generator=g) * 0.05).half()
    a = ((torch.rand(16, k, generator=g) * 2 - 1) / k ** 0.5).half()
    b = (torch.randn(nq, 16, generator=g) * 0.1).half()
    x = torch.randn(m, k, generator=g).half()
    dyq = torch.randn(m, nq, generator=g).half()
    dyk = torch.randn(m, nk, generator=g).half()
    pq, sq = quantize_nf4(wq)
    pk_, sk = quantize_nf4(wk)
    q = sharded.ShardedNF4Linear.from_quantized(pq, sq, lora_a=a, lora_b=b, scaling=scaling)
    kk = sharded.ShardedNF4Linear.from_quantized(pk_, sk)
    lo, hi = sharded.shard_rows(nq, world, rank)
    lok, hik = sharded.shard_rows(nk, world, rank)
    (yq, yk), xas = sharded.forward_local_group([q, kk], x, return_lora_inputs=True)
    grads = [dyq[:, lo:hi].contiguous(), dyk[:, lok:hik].contiguous()]
    dx, work, us = sharded.backward_dx_group([q, kk], grads, async_op=True, return_lora_inputs=True)
    work.wait()
    wgrads, works = sharded.lora_weight_grads([q, kk], x, grads, xas, us, async_op=True)
    for w_ in works:
        w_.wait()
    d_a, d_b = wgrads[0]

    full_q, full_k = oracle_weight(pq, sq), oracle_weight(pk_, sk)   # slices are exact: full weights
    y_ref, _ = nf4_oracle.lora_fwd(x, full_q, a, b, scaling)
    dxq_ref, da_ref, db_ref = nf4_oracle.lora_bwd(dyq, x, full_q, a, b, scaling)
    dx_ref = dxq_ref.float() + nf4_oracle.linear_bwd(dyk, full_k).float()
    err = nf4_oracle.max_rel_err
    out[rank] = (err(yq, y_ref[:, lo:hi]), err(yk, nf4_oracle.linear_fwd(x, full_k)[:, lok:hik]),
                 err(dx, dx_ref), err(d_a, da_ref), err(d_b, db_ref[lo:hi]), sorted(wgrads))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_lora_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        out = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_lora_worker, args=(r, world, port, out)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        for r in range(world):
            *errs, members = out[r]
            assert all(e <= 1e-2 for e in errs), errs
            assert members == [0]
