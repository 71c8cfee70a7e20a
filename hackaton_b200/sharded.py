"""Output-feature (column) sharding of the NF4 linear across the GPUs of one node.

Rank g of G holds rows [g*N/G, (g+1)*N/G) of W, quantised as an NF4 weight of its own (its own
codes, first- and second-level scales: a second-level block covers 16,384 consecutive weights
and does not end on a row boundary, so a row-sliced shard of one big quant state would not be a
clean slice of its nested array). The input X is replicated.

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


def shard_rows(n_rows: int, world: int, rank: int):
    """Row range of `rank`; N must split evenly so every shard has the same shape."""
    if n_rows % world != 0:
        raise ValueError(f"{n_rows} output features do not split evenly over {world} ranks")
    per = n_rows // world
    return rank * per, (rank + 1) * per


class ShardedNF4Linear:
    def __init__(self, packed, state, n_total: int, group=None):
        self.packed, self.state = packed, state
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_total = n_total
        self.n_local = int(state.shape[0])
        assert self.n_local * self.world == n_total

    @classmethod
    def from_full_weight(cls, weight, group=None, **quant_kwargs):
        """Quantise this rank's row shard of a full [N, K] weight."""
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        lo, hi = shard_rows(weight.shape[0], world, rank)
        packed, state = quantize_nf4(weight[lo:hi].contiguous(), **quant_kwargs)
        return cls(packed, state, weight.shape[0], group)

    def forward_local(self, x):
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


def forward_local_group(mods, x):
    """Output shards of several output-sharded projections that read the same x: one grouped launch,
    no exchange (their consumer is input-sharded)."""
    from .group import linear_forward_group
    return linear_forward_group(x, [(m.packed, m.state) for m in mods])


def backward_dx_group(mods, grad_shards, async_op=False):
    """dX of several output-sharded projections that read the same x: one grouped launch sums their
    local shares, one all-reduce sums over ranks. Returns (dX, work-or-None)."""
    from .group import linear_backward_dx_group
    dx = linear_backward_dx_group(list(grad_shards), [(m.packed, m.state) for m in mods])
    world = mods[0].world
    if world == 1:
        return dx, None
    return dx, dist.all_reduce(dx, group=mods[0].group, async_op=async_op)
