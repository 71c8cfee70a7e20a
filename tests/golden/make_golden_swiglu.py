"""Regenerates swiglu_small.npz from the reference's own SwiGLU kernel.

    TRITON_INTERPRET=1 python tests/golden/make_golden_swiglu.py /path/to/reference

What runs: the reference's `silu_mul_kernel` (solution/kernels.py:37-57), unmodified, on CPU
tensors under the Triton interpreter, in both of its modes (0 = forward, 1 = backward), launched
the way its `SiluMul` does (solution/kernels.py:66-91). Inputs: seeded normal fp16 values, one
ragged length (20,011: no multiple of the block or of a 16-byte vector) and one multiple of
the block size,
plus a few large-magnitude values so that both tails of the sigmoid are covered.
"""

import importlib
import os
import sys
from pathlib import Path

import numpy as np

os.environ.setdefault("TRITON_INTERPRET", "1")
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden*.py /path/to/reference")
    root = sys.argv[1]
    sys.path.insert(0, root)
    kernels = importlib.import_module("solution.kernels")
    import triton

    out = {}
    for name, n in (("ragged", 20 * 1001 - 9), ("blocks", 16 * 1024)):
        rng = np.random.default_rng(len(name) * 1000 + n % 997)
        gate = rng.standard_normal(n).astype(np.float16)
        up = rng.standard_normal(n).astype(np.float16)
        dout = rng.standard_normal(n).astype(np.float16)
        gate[:8] = np.array([-30, -12, -8, -0.0, 0.0, 8, 12, 30], dtype=np.float16)
        g, u, d = (torch.from_numpy(a) for a in (gate, up, dout))
        hidden, dgate, dup = torch.empty_like(g), torch.empty_like(g), torch.empty_like(g)
        grid = (triton.cdiv(n, kernels.ACT_BLOCK),)
        kernels.silu_mul_kernel[grid](g, u, hidden, hidden, hidden, *[hidden] * 5, n, 0, 0, 0, 0, 0.0,
                                      BLOCK=kernels.ACT_BLOCK, _c1=0, _c2=0, _c3=0)
        kernels.silu_mul_kernel[grid](d, g, u, dgate, dup, *[dup] * 5, n, 1, 0, 0, 0, 0.0,
                                      BLOCK=kernels.ACT_BLOCK, _c1=0, _c2=0, _c3=0)
        for key, val in (("gate", gate), ("up", up), ("dout", dout), ("hidden", hidden.numpy()),
                         ("dgate", dgate.numpy()), ("dup", dup.numpy())):
            out[f"{name}_{key}"] = val
        print(name, n, float(hidden.float().abs().max()), flush=True)
    np.savez_compressed(HERE / "swiglu_small.npz", **out)


if __name__ == "__main__":
    main()
