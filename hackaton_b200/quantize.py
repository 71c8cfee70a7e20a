"""NF4 quantiser in the bitsandbytes storage layout, used to make inputs for tests and benchmarks.

The kernels never call this: they consume whatever codes and scales a `QuantState` holds (the
live bitsandbytes object in a real model, or the one built here for synthetic weights). The
layout is the one the reference describes (solution/nf4.py:7-14): two 4-bit codes per byte, high
nibble first, one scale per `blocksize` consecutive weights; with `compress_statistics` the
scales are themselves stored as 8-bit codes with one fp32 scale per 256 of them plus a scalar
fp32 offset (solution/packed.py:57-79).

Both lookup tables are *inputs* of the kernels. `NF4_TABLE` is the 16-value data type published
in the QLoRA paper (Dettmers et al. 2023, arXiv:2305.14314, appendix E). `dynamic_8bit_table()`
builds a signed dynamic-exponent 8-bit table in the manner of the block-wise 8-bit optimiser
paper (Dettmers et al. 2022, arXiv:2110.02861): it stands in for `state2.code` when no
bitsandbytes object is at hand; decode parity does not depend on the table's values.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch

NF4_TABLE: Tuple[float, ...] = (
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
)


def nf4_table(device="cpu") -> torch.Tensor:
    return torch.tensor(NF4_TABLE, dtype=torch.float32, device=device)


def dynamic_8bit_table(device="cpu") -> torch.Tensor:
    """256 sorted values in [-1, 1]: seven decades, decade i holding 2**i evenly spaced steps."""
    values = [0.0, 1.0]
    for i in range(7):
        edges = torch.linspace(0.1, 1.0, 2 ** i + 1, dtype=torch.float64)
        centres = (edges[:-1] + edges[1:]) / 2
        scale = 10.0 ** (i - 6)
        values += (centres * scale).tolist()
        values += (-centres * scale).tolist()
    assert len(values) == 256
    return torch.tensor(sorted(values), dtype=torch.float32, device=device)


@dataclass
class NestedState:
    """Second-level state: scales of the 8-bit scale codes (bitsandbytes' `state2`)."""
    absmax: torch.Tensor          # fp32 [ceil(n_blocks / blocksize)]
    code: torch.Tensor            # fp32 [256]
    blocksize: int = 256


@dataclass
class QuantState:
    """The fields of bitsandbytes' `QuantState` that the reference reads
    (solution/nf4.py:55-64,69-76; solution/packed.py:71-79)."""
    absmax: torch.Tensor          # fp32 [n_blocks] when flat, uint8 [n_blocks] when nested
    code: torch.Tensor            # fp32 [16]
    shape: Tuple[int, int]
    dtype: torch.dtype = torch.float16
    blocksize: int = 64
    quant_type: str = "nf4"
    nested: bool = False
    state2: Optional[NestedState] = None
    offset: Optional[torch.Tensor] = None   # fp32 scalar tensor
    _cache: dict = field(default_factory=dict, repr=False, compare=False)

    def to(self, device):
        self.absmax = self.absmax.to(device)
        self.code = self.code.to(device)
        if self.state2 is not None:
            self.state2.absmax = self.state2.absmax.to(device)
            self.state2.code = self.state2.code.to(device)
        if self.offset is not None:
            self.offset = self.offset.to(device)
        self._cache.clear()
        return self


def _nearest_code(values: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Index of the nearest entry of a sorted table (ties go to the lower entry)."""
    mids = (table[1:] + table[:-1]) / 2
    return torch.bucketize(values, mids.to(values.device), right=False)


def quantize_blockwise_8bit(x: torch.Tensor, table: torch.Tensor, blocksize: int = 256):
    """8-bit block-wise quantisation of a flat fp32 vector: u8 codes and one fp32 scale per block."""
    n = x.numel()
    pad = (-n) % blocksize
    xp = torch.nn.functional.pad(x.float().reshape(-1), (0, pad)).view(-1, blocksize)
    absmax = xp.abs().amax(1)
    normed = xp / absmax.clamp_min(torch.finfo(torch.float32).tiny)[:, None]
    codes = _nearest_code(normed, table).to(torch.uint8).reshape(-1)[:n]
    return codes.contiguous(), absmax.contiguous()


def quantize_nf4(weight: torch.Tensor, blocksize: int = 64, compress_statistics: bool = True,
                 nested_blocksize: int = 256):
    """Quantise a 2-D weight to NF4. Returns (packed uint8 [n/2, 1], QuantState).

    Mirrors the call the reference's tests make,
    `F.quantize_4bit(weight, blocksize=64, compress_statistics=nested, quant_type="nf4")`
    (solution/test_nf4.py:14-15).
    """
    assert weight.dim() == 2
    n = weight.numel()
    assert n % blocksize == 0 and n % 2 == 0
    device = weight.device
    table = nf4_table(device)
    blocks = weight.detach().float().reshape(-1, blocksize)
    absmax = blocks.abs().amax(1)
    normed = blocks / absmax.clamp_min(torch.finfo(torch.float32).tiny)[:, None]
    codes = _nearest_code(normed, table).to(torch.uint8).reshape(-1)
    packed = ((codes[0::2] << 4) | codes[1::2]).contiguous().view(-1, 1)
    state = QuantState(absmax=absmax.contiguous(), code=table, shape=tuple(weight.shape),
                       dtype=weight.dtype, blocksize=blocksize)
    if compress_statistics:
        offset = absmax.mean()
        table2 = dynamic_8bit_table(device)
        q, absmax2 = quantize_blockwise_8bit(absmax - offset, table2, nested_blocksize)
        state.absmax = q
        state.nested = True
        state.state2 = NestedState(absmax=absmax2, code=table2, blocksize=nested_blocksize)
        state.offset = offset.reshape(())
    return packed, state
