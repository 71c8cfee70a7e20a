"""Regenerates rmsnorm_small.npz from the reference's own RMSNorm kernel.

    TRITON_INTERPRET=1 python tests/golden/make_golden_rmsnorm.py /path/to/reference

What runs: the reference's `rmsnorm_kernel` (solution/rmsnorm.py:17-49), unmodified, on CPU
tensors under the Triton interpreter, in its four modes (forward, backward, add + forward,
backward + the sum's own gradient), launched the way `RMSNorm` / `AddRMSNorm` do
(solution/rmsnorm.py:52-144), with fp32 and fp16 outputs. Shapes: 6 x 1536 (the Qwen2.5-1.5B
width) and 4 x 1000 (the reference test's odd width). Inputs: numpy's seeded PCG64 stream.
"""

import importlib
import os
import sys
from pathlib import Path

import numpy as np

os.environ.setdefault("TRITON_INTERPRET", "1")
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent
EPS = 1e-6


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden*.py /path/to/reference")
    root = sys.argv[1]
    sys.path.insert(0, root)
    ref = importlib.import_module("solution.rmsnorm")
    import triton

    out = {}
    for name, rows, hidden in (("qwen", 6, 1536), ("odd", 4, 1000)):
        rng = np.random.default_rng(rows * 10007 + hidden)
        x = torch.from_numpy(rng.standard_normal((rows, hidden)).astype(np.float32))
        w = torch.from_numpy((1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32))
        delta = torch.from_numpy(rng.standard_normal((rows, hidden)).astype(np.float16))
        dy32 = torch.from_numpy(rng.standard_normal((rows, hidden)).astype(np.float32))
        d_total = torch.from_numpy(rng.standard_normal((rows, hidden)).astype(np.float32))
        block = triton.next_power_of_2(hidden)
        kw = dict(BLOCK=block, _c1=0, _c2=0, _c3=0, num_warps=8)
        for key, val in (("x", x), ("w", w), ("delta", delta), ("dy", dy32), ("d_total", d_total)):
            out[f"{name}_{key}"] = val.numpy()
        for tag, dtype in (("f32", torch.float32), ("f16", torch.float16)):
            dy = dy32.to(dtype)
            y = torch.empty((rows, hidden), dtype=dtype)
            rstd = torch.empty(rows, dtype=torch.float32)
            ref.rmsnorm_kernel[(rows,)](x, w, y, rstd, y, x, *[x] * 4, rows, hidden, 0, 0, 0, EPS, **kw)
            dx = torch.empty_like(x)
            ref.rmsnorm_kernel[(rows,)](x, w, dy, rstd, dy, dx, *[dx] * 4, rows, hidden, 1, 0, 0, 0.0, **kw)
            total = torch.empty_like(x)
            y2 = torch.empty((rows, hidden), dtype=dtype)
            rstd2 = torch.empty(rows, dtype=torch.float32)
            ref.rmsnorm_kernel[(rows,)](x, w, y2, rstd2, delta, total, *[total] * 4, rows, hidden, 2, 0, 0,
                                        EPS, **kw)
            dx2 = torch.empty_like(x)
            ref.rmsnorm_kernel[(rows,)](total, w, dy, rstd2, dy, dx2, *[d_total] * 4, rows, hidden, 3, 0,
                                        0, 0.0, **kw)
            for key, val in (("y", y), ("rstd", rstd), ("dx", dx), ("total", total), ("y_add", y2),
                             ("rstd_add", rstd2), ("dx_add", dx2)):
                out[f"{name}_{tag}_{key}"] = val.numpy()
        print(name, rows, hidden, float(out[f"{name}_f32_y"].std()), flush=True)
    np.savez_compressed(HERE / "rmsnorm_small.npz", **out)


if __name__ == "__main__":
    main()
