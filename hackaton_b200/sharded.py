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
