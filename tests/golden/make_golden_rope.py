"""Regenerates rope_small.npz from the reference's own q/k/v rotation kernel.

    TRITON_INTERPRET=1 python tests/golden/make_golden_rope.py /path/to/reference

What runs: the reference's `qkv_kernel` (solution/attention.py:36-146) through its `QKVRotate`
autograd function (:149-192), unmodified, on CPU tensors under the Triton interpreter, forward and
backward, packed and padded layouts. Shapes: 3 sequences of lengths 5, 2, 4 padded to 6, 4 query
heads over 2 kv heads of size 64 (small on purpose: the kernel has no size-dependent branch).
Inputs: numpy's seeded PCG64 stream; fp16 projections as in the model, fp32 as in the
reference's test.
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
    ref = importlib.import_module("solution.attention")
    lengths, seq, heads, kv_heads, dim = [5, 2, 4], 6, 4, 2, 64
    batch = len(lengths)
    b_idx = torch.tensor([b for b, n in enumerate(lengths) for _ in range(n)], dtype=torch.int32)
    t_idx = torch.tensor([t for n in lengths for t in range(n)], dtype=torch.int32)
    n = b_idx.numel()
    rng = np.random.default_rng(4242)
    inv_freq = 1.0 / (1000000.0 ** (torch.arange(0, dim, 2).float() / dim))
    freqs = torch.arange(seq).float()[:, None] * inv_freq[None]
    emb = torch.cat((freqs, freqs), dim=-1)
    cos, sin = emb.cos()[None].contiguous(), emb.sin()[None].contiguous()
    out = {"b_idx": b_idx.numpy(), "t_idx": t_idx.numpy(), "cos": cos.numpy(), "sin": sin.numpy(),
           "meta": np.array([batch, seq, heads, kv_heads, dim])}
    for tag, dtype in (("f16", np.float16), ("f32", np.float32)):
        q = torch.from_numpy(rng.standard_normal((n, heads * dim)).astype(dtype)).requires_grad_()
        k = torch.from_numpy(rng.standard_normal((n, kv_heads * dim)).astype(dtype)).requires_grad_()
        v = torch.from_numpy(rng.standard_normal((n, kv_heads * dim)).astype(dtype)).requires_grad_()
        for key, val in (("q", q), ("k", k), ("v", v)):
            out[f"{tag}_{key}"] = val.detach().numpy()
        for layout, padded in (("packed", False), ("padded", True)):
            shape = (batch, heads, seq, dim) if padded else (n, heads, dim)
            grads = [torch.from_numpy(rng.standard_normal(shape).astype(np.float16)) for _ in range(3)]
            outs = ref.qkv_rotate(q, k, v, cos, sin, b_idx, t_idx, batch, seq, heads, kv_heads, padded)
            torch.autograd.backward(outs, grads)
            for key, val in zip(("qo", "ko", "vo"), outs):
                out[f"{tag}_{layout}_{key}"] = val.detach().numpy()
            for key, val in zip(("gq", "gk", "gv"), grads):
                out[f"{tag}_{layout}_{key}"] = val.numpy()
            for key, val in zip(("dq", "dk", "dv"), (q, k, v)):
                out[f"{tag}_{layout}_{key}"] = val.grad.numpy().copy()
                val.grad = None
        print(tag, float(out[f"{tag}_packed_qo"].astype(np.float32).std()), flush=True)
    np.savez_compressed(HERE / "rope_small.npz", **out)


if __name__ == "__main__":
    main()
