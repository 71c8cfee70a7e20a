"""Helpers shared by the tests: oracle decode of a (packed, state) pair and synthetic weights."""

import numpy as np
import torch

from oracle import nf4_oracle


def oracle_weight(packed, state):
    """fp16/bf16/fp32 weight of `state.shape` decoded by the CPU oracle."""
    p = packed.detach().cpu().numpy().reshape(-1)
    code16 = state.code.detach().cpu().numpy()
    if getattr(state, "nested", False):
        return nf4_oracle.dequant_nested(
            p, state.absmax.cpu().numpy(), state.state2.code.cpu().numpy(),
            state.state2.absmax.cpu().numpy(), float(state.offset.cpu()), code16,
            tuple(state.shape), state.blocksize, state.state2.blocksize, state.dtype)
    return nf4_oracle.dequant_flat(p, state.absmax.cpu().numpy(), code16, tuple(state.shape),
                                   state.blocksize, state.dtype)


def synthetic_weight(rows, cols, nested, seed=0, device="cpu", dtype=torch.float16):
    """W ~ 0.02 * N(0, 1) in fp16, quantised to NF4 (the reference's test weights,
    solution/test_nf4.py:9-16)."""
    from hackaton_b200.quantize import quantize_nf4

    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(rows, cols, generator=g) * 0.02).to(dtype)
    packed, state = quantize_nf4(w, blocksize=64, compress_statistics=nested)
    if device != "cpu":
        packed = packed.to(device)
        state.to(device)
    return packed, state


def random_case(seed, rows, cols, blocksize=64):
    """Same generator as tests/golden/make_golden.py: random codes and positive scales."""
    rng = np.random.default_rng(seed)
    n = rows * cols
    packed = rng.integers(0, 256, size=n // 2, dtype=np.uint8)
    absmax = np.exp(rng.standard_normal(n // blocksize).astype(np.float32) * 0.5
                    ).astype(np.float32) * np.float32(0.05)
    return packed, absmax
