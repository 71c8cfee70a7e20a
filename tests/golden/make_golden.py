"""Regenerates the golden vectors in this folder from the reference's own code.

Run once, in a container that holds the reference checkout (it is not needed to *use* the
fixtures):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference

What runs: the reference's `nf4_dequant_kernel` / `dequantize_nf4` (solution/nf4.py:28-77) and
its `NF4Linear` (solution/nf4.py:80-106), unmodified, on CPU tensors under the Triton
interpreter. Inputs are random codes and scales from numpy's PCG64 stream (seeded), so they
exercise all 16 codes; decode parity does not depend on how the codes were chosen.
Output types are fp16 and fp32 only: the interpreter converts fp32 to bf16 by truncation, unlike
the compiled kernel's round-to-nearest, so a bf16 vector made here would not pin anything.

Outputs:
  decode_small.npz   inputs and outputs of small decode cases (odd shapes, three dtypes)
  linear_small.npz   inputs and outputs of one linear forward + backward with bias
  decode_digests.json  sha256 of inputs and of the reference's output for full-size shapes,
                       whose inputs are regenerated from the seed at test time
"""

import hashlib
import importlib.util
import json
import os
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np

os.environ.setdefault("TRITON_INTERPRET", "1")
import torch  # noqa: E402

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from hackaton_b200.quantize import NF4_TABLE  # noqa: E402


def random_case(seed, rows, cols, blocksize=64):
    """Random packed codes and positive fp32 scales for a rows x cols weight."""
    rng = np.random.default_rng(seed)
    n = rows * cols
    packed = rng.integers(0, 256, size=n // 2, dtype=np.uint8)
    absmax = np.exp(rng.standard_normal(n // blocksize).astype(np.float32) * 0.5
                    ).astype(np.float32) * np.float32(0.05)
    return packed, absmax


def sha(array):
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def load_reference(root):
    spec = importlib.util.spec_from_file_location("ref_nf4", Path(root) / "solution" / "nf4.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def state_of(absmax, shape, dtype, blocksize=64):
    return SimpleNamespace(absmax=torch.from_numpy(absmax), code=torch.tensor(NF4_TABLE),
                           blocksize=blocksize, quant_type="nf4", nested=False,
                           shape=torch.Size(shape), dtype=dtype)


def as_numpy(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    ref = load_reference(sys.argv[1])
    table = np.asarray(NF4_TABLE, dtype=np.float32)

    small = {"table": table}
    cases = [("a", 100, 192, torch.float16, 64), ("b", 64, 256, torch.float16, 64),
             ("c", 8, 1536, torch.float16, 64), ("d", 16, 64, torch.float32, 64),
             ("e", 24, 128, torch.float16, 128)]
    for name, rows, cols, dtype, bs in cases:
        packed, absmax = random_case(100 + ord(name), rows, cols, bs)
        out = ref.dequantize_nf4(torch.from_numpy(packed), state_of(absmax, (rows, cols), dtype, bs))
        small[f"{name}_packed"], small[f"{name}_absmax"] = packed, absmax
        small[f"{name}_out"] = as_numpy(out)
        small[f"{name}_meta"] = np.array([rows, cols, bs, {torch.float16: 0, torch.bfloat16: 1,
                                                           torch.float32: 2}[dtype]])
    np.savez_compressed(HERE / "decode_small.npz", **small)

    # one linear forward + backward through the reference's autograd function
    rows, cols, m = 96, 192, 50
    packed, absmax = random_case(7, rows, cols)
    rng = np.random.default_rng(8)
    x = torch.from_numpy(rng.standard_normal((m, cols)).astype(np.float16)).requires_grad_()
    bias = torch.from_numpy((rng.standard_normal(rows) * 0.1).astype(np.float16))
    grad = torch.from_numpy(rng.standard_normal((m, rows)).astype(np.float16))
    state = state_of(absmax, (rows, cols), torch.float16)
    out = ref.nf4_linear(x, torch.from_numpy(packed).view(-1, 1).t(), bias, state)
    out.backward(grad)
    np.savez_compressed(HERE / "linear_small.npz", table=table, packed=packed, absmax=absmax,
                        x=x.detach().numpy(), bias=bias.numpy(), grad=grad.numpy(),
                        out=out.detach().numpy(), grad_x=x.grad.numpy())

    digests = {}
    for rows, cols in [(256, 1536), (1536, 1536), (1536, 8960)]:
        packed, absmax = random_case(rows * 31 + cols, rows, cols)
        out = ref.dequantize_nf4(torch.from_numpy(packed),
                                 state_of(absmax, (rows, cols), torch.float16))
        digests[f"{rows}x{cols}"] = {"seed": rows * 31 + cols, "packed_sha256": sha(packed),
                                     "absmax_sha256": sha(absmax), "out_sha256": sha(out.numpy())}
        print(rows, cols, digests[f"{rows}x{cols}"]["out_sha256"][:16], flush=True)
    (HERE / "decode_digests.json").write_text(json.dumps(digests, indent=1) + "\n")


if __name__ == "__main__":
    main()
