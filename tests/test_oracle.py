"""CPU: the oracle against the golden vectors made with the reference's own code
(tests/golden/make_golden.py), and the C restatement against the numpy one."""

import ctypes
import hashlib
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import nf4_oracle
from tests.util import random_case, synthetic_weight, oracle_weight

GOLDEN = Path(__file__).resolve().parent / "golden"
DTYPES = {0: torch.float16, 1: torch.bfloat16, 2: torch.float32}


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def to_numpy(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


@pytest.mark.parametrize("name", list("abcde"))
def test_flat_decode_matches_reference_kernel(name):
    g = np.load(GOLDEN / "decode_small.npz")
    rows, cols, bs, dt = (int(v) for v in g[f"{name}_meta"])
    out = nf4_oracle.dequant_flat(g[f"{name}_packed"], g[f"{name}_absmax"], g["table"],
                                  (rows, cols), bs, DTYPES[dt])
    assert np.array_equal(to_numpy(out), g[f"{name}_out"])


@pytest.mark.parametrize("shape", ["256x1536", "1536x1536", "1536x8960"])
def test_flat_decode_digest_full_size(shape):
    d = json.loads((GOLDEN / "decode_digests.json").read_text())[shape]
    rows, cols = (int(v) for v in shape.split("x"))
    packed, absmax = random_case(d["seed"], rows, cols)
    assert sha(packed) == d["packed_sha256"] and sha(absmax) == d["absmax_sha256"], \
        "numpy's seeded stream changed: regenerate tests/golden"
    from hackaton_b200.quantize import NF4_TABLE
    out = nf4_oracle.dequant_flat(packed, absmax, np.asarray(NF4_TABLE, np.float32), (rows, cols))
    assert sha(out.numpy()) == d["out_sha256"]


def test_linear_matches_reference_autograd_function():
    g = np.load(GOLDEN / "linear_small.npz")
    w = nf4_oracle.dequant_flat(g["packed"], g["absmax"], g["table"], (96, 192))
    x, grad, bias = (torch.from_numpy(g[k]) for k in ("x", "grad", "bias"))
    out = nf4_oracle.linear_fwd(x, w, bias)
    gx = nf4_oracle.linear_bwd(grad, w)
    torch.testing.assert_close(out, torch.from_numpy(g["out"]), rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(gx, torch.from_numpy(g["grad_x"]), rtol=2e-3, atol=2e-3)


def test_nested_scales_are_two_roundings():
    rng = np.random.default_rng(3)
    q = rng.integers(0, 256, size=1000, dtype=np.uint8)
    code2 = np.sort(rng.uniform(-1, 1, 256)).astype(np.float32)
    absmax2 = rng.uniform(0.01, 0.1, 4).astype(np.float32)
    flat = nf4_oracle.flatten_absmax(q, code2, absmax2, 0.0371, 256)
    want = (code2[q] * absmax2[np.arange(1000) // 256]).astype(np.float32) + np.float32(0.0371)
    assert flat.dtype == np.float32 and np.array_equal(flat, want)


@pytest.fixture(scope="module")
def c_oracle():
    folder = Path(__file__).resolve().parents[1] / "oracle"
    subprocess.run(["make", "-C", str(folder), "libnf4_oracle.so"], check=True,
                   stdout=subprocess.DEVNULL)
    return ctypes.CDLL(str(folder / "libnf4_oracle.so"))


@pytest.mark.parametrize("nested", [False, True])
def test_c_restatement_equals_numpy(c_oracle, nested):
    packed, state = synthetic_weight(96, 320, nested, seed=5)
    want = oracle_weight(packed, state).numpy().view(np.uint16)
    n = 96 * 320
    out = np.empty(n, dtype=np.uint16)
    p = packed.numpy().reshape(-1)
    ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    code16 = state.code.numpy()
    if nested:
        a, c2, a2 = state.absmax.numpy(), state.state2.code.numpy(), state.state2.absmax.numpy()
        c_oracle.oracle_dequant_nested_f16(ptr(p), ptr(a), ptr(c2), ptr(a2),
                                           ctypes.c_float(float(state.offset)), ptr(code16),
                                           ctypes.c_int64(n), 64, 256, ptr(out))
    else:
        a = state.absmax.numpy()
        c_oracle.oracle_dequant_flat_f16(ptr(p), ptr(a), ptr(code16), ctypes.c_int64(n), 64,
                                         ptr(out))
    assert np.array_equal(out, want.reshape(-1))


def test_quantiser_round_trip_error_is_small():
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(64, 256, generator=g) * 0.02).half()
    for nested in (False, True):
        from hackaton_b200.quantize import quantize_nf4
        packed, state = quantize_nf4(w, compress_statistics=nested)
        assert packed.shape == (64 * 256 // 2, 1) and packed.dtype == torch.uint8
        back = oracle_weight(packed, state)
        err = (back.float() - w.float()).abs().max() / w.float().abs().max()
        assert err < 0.2


@pytest.mark.parametrize("nested", [False, True])
def test_threaded_variant_equals_numpy(nested):
    packed, state = synthetic_weight(96, 320, nested, seed=6)
    kw = {}
    if nested:
        kw = dict(code2=state.state2.code, absmax2=state.state2.absmax, offset=state.offset)
    got = nf4_oracle.dequant_torch(packed, state.absmax, state.code, (96, 320), **kw)
    assert torch.equal(got.view(torch.int16), oracle_weight(packed, state).view(torch.int16))


@pytest.mark.parametrize("name", ["ragged", "blocks"])
def test_swiglu_matches_reference_kernel(name):
    """The oracle's SwiGLU against the outputs of the reference's silu_mul_kernel (both modes,
    made under the Triton interpreter: tests/golden/make_golden_swiglu.py). Same fp32 formula,
    but libm's and the interpreter's exp may differ in the last bit, so: at most one fp16 step,
    and hardly anywhere."""
    z = np.load(GOLDEN / "swiglu_small.npz")
    gate, up, dout = (torch.from_numpy(z[f"{name}_{k}"]) for k in ("gate", "up", "dout"))
    got = {"hidden": nf4_oracle.swiglu_fwd(gate, up)}
    got["dgate"], got["dup"] = nf4_oracle.swiglu_bwd(dout, gate, up)
    for key, val in got.items():
        want = torch.from_numpy(z[f"{name}_{key}"])
        steps = (val.view(torch.int16).int() - want.view(torch.int16).int()).abs()
        same_sign = (val.view(torch.int16) ^ want.view(torch.int16)) >= 0
        assert bool(((steps <= 1) | ~same_sign & (val.abs() + want.abs() < 1e-6)).all()), key
        assert float((steps > 0).float().mean()) < 1e-3, key


@pytest.mark.parametrize("name", ["qwen", "odd"])
@pytest.mark.parametrize("tag", ["f32", "f16"])
def test_rmsnorm_matches_reference_kernel(name, tag):
    """The oracle's RMSNorm against the reference's rmsnorm_kernel in its four modes
    (tests/golden/make_golden_rmsnorm.py). The row sums are taken in another order than the
    interpreter's tree, so: fp32 results within 2e-6 relative, fp16 outputs within one step."""
    z = np.load(GOLDEN / "rmsnorm_small.npz")
    t = lambda key: torch.from_numpy(z[f"{name}_{key}"])
    dtype = torch.float32 if tag == "f32" else torch.float16
    x, w, delta, d_total = t("x"), t("w"), t("delta"), t("d_total")
    dy = t("dy").to(dtype)
    tol = dict(rtol=2e-6, atol=2e-6) if tag == "f32" else dict(rtol=1e-3, atol=1e-3)
    y, rstd, _ = nf4_oracle.rmsnorm_fwd(x, w, 1e-6, None, dtype)
    torch.testing.assert_close(y.float(), t(f"{tag}_y").float(), **tol)
    torch.testing.assert_close(rstd, t(f"{tag}_rstd"), rtol=2e-6, atol=0)
    torch.testing.assert_close(nf4_oracle.rmsnorm_bwd(x, w, rstd, dy), t(f"{tag}_dx"), rtol=2e-5, atol=2e-6)
    y2, rstd2, total = nf4_oracle.rmsnorm_fwd(x, w, 1e-6, delta, dtype)
    assert torch.equal(total, t(f"{tag}_total"))          # the same fp32 addition
    torch.testing.assert_close(y2.float(), t(f"{tag}_y_add").float(), **tol)
    torch.testing.assert_close(nf4_oracle.rmsnorm_bwd(total, w, rstd2, dy, d_total), t(f"{tag}_dx_add"),
                               rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("tag", ["f16", "f32"])
@pytest.mark.parametrize("layout", ["packed", "padded"])
def test_qkv_rotate_matches_reference_kernel(tag, layout):
    """The oracle's rotation + GQA expansion against the reference's qkv_kernel run through its
    QKVRotate (tests/golden/make_golden_rope.py). Products and sums may be contracted differently
    (one fp32 rounding), so fp16 outputs may differ by one step in a few places."""
    z = np.load(GOLDEN / "rope_small.npz")
    t = lambda key: torch.from_numpy(z[key])
    batch, seq, heads, kv_heads, dim = (int(x) for x in z["meta"])
    padded = layout == "padded"
    args = (t("cos"), t("sin"), t("b_idx"), t("t_idx"))
    outs = nf4_oracle.qkv_rotate_fwd(t(f"{tag}_q"), t(f"{tag}_k"), t(f"{tag}_v"), *args, batch, seq,
                                     heads, kv_heads, padded)
    for got, key in zip(outs, ("qo", "ko", "vo")):
        want = t(f"{tag}_{layout}_{key}")
        assert got.shape == want.shape and got.dtype == want.dtype
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-3, atol=1e-3)
    assert torch.equal(outs[2], t(f"{tag}_{layout}_vo"))        # v is only copied
    dtype = torch.float16 if tag == "f16" else torch.float32
    grads = nf4_oracle.qkv_rotate_bwd(*(t(f"{tag}_{layout}_{k}") for k in ("gq", "gk", "gv")), *args,
                                      heads, kv_heads, padded, dtype)
    tol = dict(rtol=2e-3, atol=2e-3) if tag == "f16" else dict(rtol=1e-5, atol=1e-5)
    for got, key in zip(grads, ("dq", "dk", "dv")):
        want = t(f"{tag}_{layout}_{key}")
        assert got.shape == want.shape and got.dtype == want.dtype
        torch.testing.assert_close(got.float(), want.float(), **tol)


@pytest.mark.parametrize("name", ["ragged", "blocks"])
@pytest.mark.parametrize("tag", ["f16", "f32"])
def test_cross_entropy_matches_reference_kernel(name, tag):
    """The oracle's cross-entropy against the reference's ce_kernel, both passes
    (tests/golden/make_golden_ce.py): fp32 sums in another order, the argmax exact."""
    z = np.load(GOLDEN / "ce_small.npz")
    t = lambda key: torch.from_numpy(z[f"{name}_{tag}_{key}"])
    logits, targets = t("logits"), torch.from_numpy(z[f"{name}_targets"])
    lse, loss, entropy, argmax = nf4_oracle.ce_stats(logits, targets)
    torch.testing.assert_close(lse, t("lse"), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(loss, t("loss"), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(entropy, t("entropy"), rtol=1e-4, atol=1e-4)
    assert torch.equal(argmax, t("argmax"))
    assert float(lse[2]) == 0.0 and float(loss[2]) == 0.0          # the ignored row
    grad = nf4_oracle.ce_grad(logits, targets, t("lse"), 0.37)
    tol = dict(rtol=2e-3, atol=1e-6) if tag == "f16" else dict(rtol=1e-4, atol=1e-7)
    torch.testing.assert_close(grad.float(), t("grad").float(), **tol)
    assert not bool(t("grad")[2].any())
