"""GPU: standalone decode through the C ABI, bit-equal to the oracle and to the reference's
golden vectors (the shapes of the reference's solution/test_nf4.py:28-43 plus odd ones)."""

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from hackaton_b200.quantize import NF4_TABLE, QuantState, nf4_table
from tests.util import oracle_weight, random_case, synthetic_weight

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
DTYPES = {0: torch.float16, 1: torch.bfloat16, 2: torch.float32}


def bits(t):
    t = t.detach().cpu()
    return t.view(torch.int16) if t.element_size() == 2 else t.view(torch.int32)


@pytest.mark.parametrize("rows,cols,nested", [(256, 1536, False), (1536, 8960, True),
                                              (8960, 1536, True), (100, 192, False),
                                              (100, 192, True), (8, 64, True), (3, 64, False)])
def test_decode_is_bit_identical_to_oracle(cuda_lib, rows, cols, nested):
    from hackaton_b200 import can_dequantize, dequantize_nf4

    packed, state = synthetic_weight(rows, cols, nested, seed=rows + cols, device="cuda")
    assert can_dequantize(packed, state)
    mine = dequantize_nf4(packed, state)
    want = oracle_weight(packed, state)
    assert mine.dtype == want.dtype and tuple(mine.shape) == (rows, cols)
    assert torch.equal(bits(mine), bits(want))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("nested", [False, True])
def test_decode_output_types(cuda_lib, dtype, nested):
    from hackaton_b200 import dequantize_nf4

    packed, state = synthetic_weight(64, 320, nested, seed=11, device="cuda")
    state.dtype = dtype
    mine = dequantize_nf4(packed, state)
    assert mine.dtype == dtype
    assert torch.equal(bits(mine), bits(oracle_weight(packed, state)))


@pytest.mark.parametrize("name", list("abcde"))
def test_decode_matches_reference_golden(cuda_lib, name):
    from hackaton_b200 import dequantize_nf4

    g = np.load(GOLDEN / "decode_small.npz")
    rows, cols, bs, dt = (int(v) for v in g[f"{name}_meta"])
    state = QuantState(absmax=torch.from_numpy(g[f"{name}_absmax"]).cuda(),
                       code=torch.from_numpy(g["table"]).cuda(), shape=(rows, cols),
                       dtype=DTYPES[dt], blocksize=bs)
    mine = dequantize_nf4(torch.from_numpy(g[f"{name}_packed"]).cuda(), state)
    got = mine.cpu()
    got = got.view(torch.int16).numpy().view(np.uint16) if dt == 1 else got.numpy()
    assert np.array_equal(got, g[f"{name}_out"])


@pytest.mark.parametrize("shape", ["256x1536", "1536x1536", "1536x8960"])
def test_decode_digest_full_size(cuda_lib, shape):
    from hackaton_b200 import dequantize_nf4

    d = json.loads((GOLDEN / "decode_digests.json").read_text())[shape]
    rows, cols = (int(v) for v in shape.split("x"))
    packed, absmax = random_case(d["seed"], rows, cols)
    state = QuantState(absmax=torch.from_numpy(absmax).cuda(), code=nf4_table("cuda"),
                       shape=(rows, cols))
    out = dequantize_nf4(torch.from_numpy(packed).cuda(), state).cpu().numpy()
    assert hashlib.sha256(out.tobytes()).hexdigest() == d["out_sha256"]


def test_table_is_an_input(cuda_lib):
    """Any 16-entry table decodes through the same path (the kernel takes it as a pointer)."""
    from hackaton_b200 import dequantize_nf4

    packed, state = synthetic_weight(32, 128, True, seed=2, device="cuda")
    state.code = torch.linspace(-3, 5, 16, device="cuda")
    assert torch.equal(bits(dequantize_nf4(packed, state)), bits(oracle_weight(packed, state)))


def test_rejects_what_it_cannot_decode(cuda_lib):
    from hackaton_b200 import can_dequantize, dequantize_nf4

    packed, state = synthetic_weight(32, 128, False, seed=2, device="cuda")
    state.quant_type = "fp4"
    assert not can_dequantize(packed, state)
    with pytest.raises(ValueError):
        dequantize_nf4(packed, state)
    state.quant_type = "nf4"
    assert not can_dequantize(packed.cpu(), state)


@pytest.mark.parametrize("nested", [True, False])
def test_store_routes_and_grid_stride(cuda_lib, nested):
    """16-bit outputs leave through a staging area and one bulk copy per tile, fp32 outputs with
    per-thread stores; a weight with more tiles than resident CTAs (18944 x 3584: 4145 tiles for
    888 CTAs) makes every CTA reuse its staging area. The fp32 result rounded to fp16 is the fp16
    result (one product, one rounding), and both ends of the walk equal the oracle."""
    import copy

    from hackaton_b200 import dequantize_nf4
    from tests.util import oracle_weight, synthetic_weight

    rows, cols = 18944, 3584
    packed, state = synthetic_weight(rows, cols, nested, seed=21, device="cuda")
    half = dequantize_nf4(packed, state)
    state32 = copy.copy(state)
    state32.dtype = torch.float32
    full = dequantize_nf4(packed, state32)
    assert full.dtype == torch.float32 and torch.equal(full.half(), half)
    want = oracle_weight(packed, state)
    for sl in (slice(0, 64), slice(rows - 64, rows)):
        assert torch.equal(half[sl].cpu(), want[sl])
    assert cuda_lib.device_status() == 0
