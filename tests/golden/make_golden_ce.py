"""Regenerates ce_small.npz from the reference's own cross-entropy kernel.

    TRITON_INTERPRET=1 python tests/golden/make_golden_ce.py /path/to/reference

What runs: the reference's `ce_kernel` (solution/kernels.py:106-170) through its `ce_stats` (all
four outputs) and `ce_grad` (solution/kernels.py:173-204), unmodified, on CPU tensors under the
Triton interpreter. Shapes: 4 rows of 9,001 logits (more than two blocks of 4,096, not a multiple
of 8) and 3 rows of 4,096, fp16 and fp32; one ignored row (target -100) in each; one row with its
maximum repeated (the argmax must be the first). Inputs: numpy's seeded PCG64 stream, scaled so
that a few logits dominate as in a trained model.
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
    ref = importlib.import_module("solution.kernels")
    out = {}
    for name, rows, vocab in (("ragged", 4, 9001), ("blocks", 3, 4096)):
        rng = np.random.default_rng(rows * 131 + vocab)
        base = rng.standard_normal((rows, vocab)).astype(np.float32) * 3.0
        base[1, 17] = base[1, 5000 % vocab] = base[1].max() + 1.0        # a repeated maximum
        targets = rng.integers(0, vocab, size=rows).astype(np.int64)
        targets[2] = -100
        out[f"{name}_targets"] = targets
        for tag, dtype in (("f16", torch.float16), ("f32", torch.float32)):
            logits = torch.from_numpy(base).to(dtype)
            t = torch.from_numpy(targets)
            lse = torch.empty(rows, dtype=torch.float32)
            loss, entropy = torch.empty_like(lse), torch.empty_like(lse)
            argmax = torch.empty(rows, dtype=torch.int64)
            ref.ce_stats(logits, t, True, out=(lse, loss, entropy, argmax))
            scale = torch.tensor([0.37], dtype=torch.float32)
            grad = torch.empty_like(logits)
            ref.ce_grad(logits, t, lse, scale, grad)
            for key, val in (("logits", logits), ("lse", lse), ("loss", loss), ("entropy", entropy),
                             ("argmax", argmax), ("grad", grad)):
                out[f"{name}_{tag}_{key}"] = val.numpy()
        print(name, rows, vocab, out[f"{name}_f16_loss"], flush=True)
    np.savez_compressed(HERE / "ce_small.npz", **out)


if __name__ == "__main__":
    main()
