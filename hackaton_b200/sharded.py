"""Output-feature (column) sharding of the NF4 linear across the GPUs of one node.

Rank g of G holds rows [g*N/G, (g+1)*N/G) of W as an NF4 weight of its own: either quantised
from the rank's slice of an fp16 weight (`from_full_weight`) or cut out of an already quantised
weight (`from_quantized`, see below). The input X is replicated.

  forward : Y_g = X . W_gᵀ on each rank (fused kernel), then an NCCL all-gather of the shards.
            The gathered tensor is shard-major, [G, M, N/G]; `row_major()` rearranges it to
            [M, N] when a consumer needs that layout.
  backward: dX_g = dY[:, shard g] . W_g on each rank (fused kernel), then an NCCL all-reduce
            (sum) of the partial input gradients.

Pairing (`InputShardedNF4Linear`): a projection that consumes what output-sharded projections
produce (o after q/k/v + attention over the rank's heads, down after gate/up + SwiGLU on the
rank's columns) holds COLUMNS [g*K/G, (g+1)*K/G) of its W instead. Its input is then exactly the
shard the rank already has, so nothing is gathered:

  forward : Y = sum_g X_g . W_gᵀ: local GEMM on the shard, then one all-reduce of [M, N]
  backward: dX_g = dY . W_g is this rank's shard of dX: no exchange at all

and the output-sharded members need no all-gather either (`forward_local`), only the all-reduce
of their summed dX (`backward_dx_group`). Per decoder layer that is four all-reduces of
[M, hidden] instead of seven all-gathers and seven all-reduces (6x fewer bytes at the 7B shapes).
Shard boundaries along K fall on multiples of 64, so every shard is a whole number of NF4 blocks.

LoRA on an output-sharded projection (q, v): A [16, K] is replicated, B [N, 16] is split by rows
with W. The forward's rank-16 term and the rank's share of dX ride in the same fused launches
(u_g = s . dY_g . B_g, and sum_g u_g . A is part of the one all-reduce of dX); dB_g is local, and
dA = sum_g u_gᵀ . X is a [16, K] fp32 all-reduce (`lora_weight_grads`).

Sharding an existing quantised weight (`slice_rows` / `slice_cols`): shard boundaries fall on
whole 64-weight blocks, so the codes and the first-level scales of a shard are exact slices of
the full weight's; the second-level blocks (256 first-level scales) do not end on shard
boundaries, so the shard carries its first-level scales flattened to fp32 (the reference's own
layout, solution/packed.py:57-79) and decodes to exactly the matching slice of the full weight.
`from_full_weight` instead quantises the rank's slice of an fp16 weight on its own (other
second-level blocks and another offset: close to, but not bit-equal to, the single-GPU weight).

Precision of the input-sharded forward: every rank rounds its partial sum to fp16 before the
all-reduce (the single-GPU kernel rounds the full fp32 sum once), so the result carries up to G
extra half-ulp roundings: relative error <= G * 2^-11 of the largest partial, about 4e-3 at G = 8,
inside the 1e-2 bound the fused linear is held to.

The reference is single-GPU (harness/common.py:39); this is the one parallel strategy the
B200 build adds. Collectives run through torch.distributed (NCCL over NVLink/NVSwitch); with
`async_op=True` the transfer of one projection overlaps the GEMM of the next.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .nf4 import linear_backward_dx, linear_forward
from .quantize import quantize_nf4


def reserve_comm_sms(n_sms: int) -> int:
    """Keeps `n_sms` SMs of the current device out of the fused GEMMs' persistent grids, so that the
    NCCL kernel of one projection can run next to the GEMM of the next one (a grid that occupies
    every SM leaves a collective nothing to start on). 0 gives all SMs back. Returns the number of
    SMs the GEMMs use from now on. Pair it with NCCL's own CTA cap (`NCCL_MAX_CTAS`)."""
    from . import _lib

    total = _lib.query(torch.cuda.current_device()).sm_count
    use = total if n_sms <= 0 else max(2, total - int(n_sms))
    _lib.set_sm_limit(0 if use == total else use)
    return use


def _flat_scales(state):
    """fp32 first-level scales of a quant state (two-level states decoded as the reference's
    `_flatten_quant_states` does: code2[u8] * absmax2[i // 256], then + offset; two roundings)."""
    if not getattr(state, "nested", False):
        return state.absmax.float()
    s2 = state.state2
    idx = torch.arange(state.absmax.numel(), device=state.absmax.device) // int(s2.blocksize)
    flat = s2.code.float()[state.absmax.long()] * s2.absmax.float()[idx]
    return flat + state.offset.float()


def slice_rows(packed, state, lo: int, hi: int):
    """(packed, state) of rows [lo, hi) of an existing NF4 weight, decoding to exactly those rows
    of the full weight. K must be a multiple of the block size."""
    from .quantize import QuantState

    n, k = int(state.shape[0]), int(state.shape[1])
    bs = int(state.blocksize)
    if k % bs != 0 or k % 2 != 0:
        raise ValueError(f"{k} input features are not whole NF4 blocks of {bs}")
    codes = packed.reshape(n, k // 2)[lo:hi].contiguous().reshape(-1, 1)
    scales = _flat_scales(state).reshape(n, k // bs)[lo:hi].contiguous().reshape(-1)
    return codes, QuantState(absmax=scales, code=state.code, shape=(hi - lo, k), dtype=state.dtype,
                             blocksize=bs)


def slice_cols(packed, state, lo: int, hi: int):
    """(packed, state) of input features [lo, hi) of an existing NF4 weight; lo and hi must be
    multiples of the block size."""
    from .quantize import QuantState

    n, k = int(state.shape[0]), int(state.shape[1])
    bs = int(state.blocksize)
    if lo % bs != 0 or hi % bs != 0 or k % bs != 0:
        raise ValueError(f"columns [{lo}, {hi}) of {k} do not fall on NF4 blocks of {bs}")
    codes = packed.reshape(n, k // 2)[:, lo // 2:hi // 2].contiguous().reshape(-1, 1)
    scales = _flat_scales(state).reshape(n, k // bs)[:, lo // bs:hi // bs].contiguous().reshape(-1)
    return codes, QuantState(absmax=scales, code=state.code, shape=(n, hi - lo), dtype=state.dtype,
                             blocksize=bs)


def shard_rows(n_rows: int, world: int, rank: int):
    """Row range of `rank`; N must split evenly so every shard has the same shape."""
    if n_rows % world != 0:
        raise ValueError(f"{n_rows} output features do not split evenly over {world} ranks")
    per = n_rows // world
    return rank * per, (rank + 1) * per


class ShardedNF4Linear:
    def __init__(self, packed, state, n_total: int, group=None, lora_a=None, lora_b=None,
                 scaling: float = 1.0):
        self.packed, self.state = packed, state
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_total = n_total
        self.n_local = int(state.shape[0])
        assert self.n_local * self.world == n_total
        if (lora_a is None) != (lora_b is None):
            raise ValueError("a sharded projection needs both LoRA factors or none")
        if lora_b is not None and lora_b.shape[0] != self.n_local:
            raise ValueError("lora_b must hold this rank's rows of B")
        self.lora_a, self.lora_b, self.scaling = lora_a, lora_b, float(scaling)

    @classmethod
    def from_quantized(cls, packed, state, group=None, lora_a=None, lora_b=None, scaling=1.0):
        """This rank's row shard of an already quantised full weight (e.g. one read from a 4-bit
        checkpoint): decodes to exactly the matching rows of the full weight. `lora_b`, if given,
        is the full [N, 16] factor; the rank keeps its rows."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        lo, hi = shard_rows(int(state.shape[0]), world, rank)
        p, st = slice_rows(packed, state, lo, hi)
        b = None if lora_b is None else lora_b[lo:hi].contiguous()
        return cls(p, st, int(state.shape[0]), group, lora_a, b, scaling)

    @classmethod
    def from_full_weight(cls, weight, group=None, **quant_kwargs):
        """Quantise this rank's row shard of a full [N, K] weight."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        lo, hi = shard_rows(weight.shape[0], world, rank)
        packed, state = quantize_nf4(weight[lo:hi].contiguous(), **quant_kwargs)
        return cls(packed, state, weight.shape[0], group)

    def forward_local(self, x):
        if self.lora_a is not None:
            return forward_local_group([self], x)[0]
        return linear_forward(x, self.packed, None, self.state)

    def forward(self, x, async_op=False):
        """Returns (gathered [G, M, N/G], work-or-None)."""
        y = self.forward_local(x)
        if self.world == 1:
            return y.reshape(1, -1, y.shape[-1]), None
        y2 = y.reshape(-1, y.shape[-1])
        flat = torch.empty((self.world * y2.shape[0], y2.shape[1]), dtype=y.dtype, device=y.device)
        work = dist.all_gather_into_tensor(flat, y2, group=self.group, async_op=async_op)
        return flat.view(self.world, y2.shape[0], y2.shape[1]), work

    def backward_dx(self, grad_shard, async_op=False):
        """grad_shard: this rank's [M, N/G] slice of dY. Returns (dX summed over ranks, work)."""
        if self.lora_a is not None:
            return backward_dx_group([self], [grad_shard], async_op=async_op)
        dx = linear_backward_dx(grad_shard, self.packed, self.state)
        if self.world == 1:
            return dx, None
        work = dist.all_reduce(dx, group=self.group, async_op=async_op)
        return dx, work

    @staticmethod
    def row_major(gathered):
        """[G, M, N/G] -> [M, N]."""
        g, m, n = gathered.shape
        return gathered.permute(1, 0, 2).reshape(m, g * n)


class InputShardedNF4Linear:
    """Rank g holds columns [g*K/G, (g+1)*K/G) of W (its input features), quantised as an NF4
    weight of its own; the input arrives as the matching [M, K/G] shard."""

    def __init__(self, packed, state, k_total: int, group=None):
        self.packed, self.state = packed, state
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.k_total = k_total
        self.k_local = int(state.shape[1])
        assert self.k_local * self.world == k_total
        if self.k_local % 64 != 0:
            raise ValueError(f"{k_total} input features over {self.world} ranks: shards of {self.k_local} "
                             "columns are not whole NF4 blocks of 64")

    @classmethod
    def from_quantized(cls, packed, state, group=None):
        """This rank's column shard of an already quantised full weight."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        lo, hi = shard_rows(int(state.shape[1]), world, rank)
        p, st = slice_cols(packed, state, lo, hi)
        return cls(p, st, int(state.shape[1]), group)

    @classmethod
    def from_full_weight(cls, weight, group=None, **quant_kwargs):
        """Quantise this rank's column shard of a full [N, K] weight."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        lo, hi = shard_rows(weight.shape[1], world, rank)
        packed, state = quantize_nf4(weight[:, lo:hi].contiguous(), **quant_kwargs)
        return cls(packed, state, weight.shape[1], group)

    def forward_local(self, x_shard):
        return linear_forward(x_shard, self.packed, None, self.state)

    def forward(self, x_shard, async_op=False):
        """x_shard: [M, K/G]. Returns (Y summed over ranks [M, N], work-or-None)."""
        y = self.forward_local(x_shard)
        if self.world == 1:
            return y, None
        return y, dist.all_reduce(y, group=self.group, async_op=async_op)

    def backward_dx(self, grad, async_op=False):
        """grad: the full [M, N] dY. Returns (this rank's [M, K/G] shard of dX, None)."""
        return linear_backward_dx(grad, self.packed, self.state), None


def _lora_members(mods):
    return [i for i, m in enumerate(mods) if getattr(m, "lora_a", None) is not None]


def forward_local_group(mods, x, return_lora_inputs=False):
    """Output shards of several output-sharded projections that read the same x: one grouped launch,
    no exchange (their consumer is input-sharded). Members with LoRA get their rank-16 term in the
    same launch; with `return_lora_inputs` the per-member s . x . Aᵀ (needed for dB) come back too."""
    from .group import linear_forward_group
    from .lora import lora_down_batch

    xas = [None] * len(mods)
    with_lora = _lora_members(mods)
    if with_lora:
        downs = lora_down_batch([x] * len(with_lora), [mods[i].lora_a for i in with_lora], True,
                                [mods[i].scaling for i in with_lora])
        for i, xa in zip(with_lora, downs):
            xas[i] = xa
    outs = linear_forward_group(x, [(m.packed, m.state) for m in mods], None, xas,
                                [getattr(m, "lora_b", None) for m in mods])
    return (outs, xas) if return_lora_inputs else outs


def backward_dx_group(mods, grad_shards, async_op=False, return_lora_inputs=False):
    """dX of several output-sharded projections that read the same x: one grouped launch sums their
    local shares (LoRA shares included), one all-reduce sums over ranks. Returns (dX, work-or-None)
    and, with `return_lora_inputs`, the per-member s . dY_g . B_g (needed for dA)."""
    from .group import linear_backward_dx_group
    from .lora import lora_down_batch

    grad_shards = list(grad_shards)
    us = [None] * len(mods)
    with_lora = _lora_members(mods)
    if with_lora:
        downs = lora_down_batch([grad_shards[i] for i in with_lora], [mods[i].lora_b for i in with_lora],
                                False, [mods[i].scaling for i in with_lora])
        for i, u in zip(with_lora, downs):
            us[i] = u
    dx = linear_backward_dx_group(grad_shards, [(m.packed, m.state) for m in mods], us,
                                  [getattr(m, "lora_a", None) for m in mods])
    world = mods[0].world
    work = None if world == 1 else dist.all_reduce(dx, group=mods[0].group, async_op=async_op)
    return (dx, work, us) if return_lora_inputs else (dx, work)


def lora_weight_grads(mods, x, grad_shards, xas, us, async_op=False):
    """fp32 gradients of the LoRA factors of the members that have them, in one launch:
    dA = sum over ranks of u_gᵀ . x ([16, K], all-reduced: A is replicated), dB_g = dY_gᵀ . xa
    ([N/G, 16], local: B is sharded with W). Returns ({member index: (dA, dB)}, [works])."""
    from .lora import lora_grad_batch

    with_lora = _lora_members(mods)
    if not with_lora:
        return {}, []
    zs, ss, rank_major = [], [], []
    for i in with_lora:
        zs += [x, grad_shards[i]]
        ss += [us[i], xas[i]]
        rank_major += [True, False]
    res = lora_grad_batch(zs, ss, rank_major)
    out, works = {}, []
    for j, i in enumerate(with_lora):
        d_a, d_b = res[2 * j], res[2 * j + 1]
        if mods[i].world > 1:
            works.append(dist.all_reduce(d_a, group=mods[i].group, async_op=async_op))
        out[i] = (d_a, d_b)
    return out, [w for w in works if w is not None]
