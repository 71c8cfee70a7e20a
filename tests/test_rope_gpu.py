"""GPU: rotary embedding + grouped-query expansion through the C ABI against the reference
kernel's golden vectors, the oracle and transformers' formula (the reference's own test,
solution/test_attention.py:40-81)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import nf4_oracle

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("tag", ["f16", "f32"])
@pytest.mark.parametrize("layout", ["packed", "padded"])
def test_matches_reference_kernel(cuda_lib, tag, layout):
    from hackaton_b200.rope import qkv_rotate

    z = np.load(GOLDEN / "rope_small.npz")
    t = lambda key: torch.from_numpy(z[key]).cuda()
    batch, seq, heads, kv_heads, dim = (int(x) for x in z["meta"])
    padded = layout == "padded"
    q, k, v = (t(f"{tag}_{n}").requires_grad_() for n in ("q", "k", "v"))
    outs = qkv_rotate(q, k, v, t("cos"), t("sin"), t("b_idx"), t("t_idx"), batch, seq, heads, kv_heads, padded)
    torch.autograd.backward(outs, [t(f"{tag}_{layout}_{g}") for g in ("gq", "gk", "gv")])
    for got, key in zip(outs, ("qo", "ko", "vo")):
        want = t(f"{tag}_{layout}_{key}")
        assert got.shape == want.shape and got.dtype == want.dtype
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-3, atol=1e-3)
    assert torch.equal(outs[2], t(f"{tag}_{layout}_vo"))
    tol = dict(rtol=2e-3, atol=2e-3) if tag == "f16" else dict(rtol=1e-5, atol=1e-5)
    for got, key in zip((q.grad, k.grad, v.grad), ("dq", "dk", "dv")):
        want = t(f"{tag}_{layout}_{key}")
        assert got.shape == want.shape and got.dtype == want.dtype
        torch.testing.assert_close(got.float(), want.float(), **tol)
    cuda_lib.device_status()


def token_maps(lengths, seq):
    real = torch.zeros(len(lengths), seq, dtype=torch.bool, device="cuda")
    for i, n in enumerate(lengths):
        real[i, :n] = True
    rows = torch.nonzero(real.reshape(-1), as_tuple=True)[0]
    return rows, (rows // seq).to(torch.int32), (rows % seq).to(torch.int32)


def rotate_half(x):
    return torch.cat((-x[..., x.shape[-1] // 2:], x[..., : x.shape[-1] // 2]), dim=-1)


def transformers_path(q, k, v, cos, sin, heads, kv_heads):
    """What Qwen2 attention does to the projections: view as heads, rotate, repeat kv heads."""
    b, t, _ = q.shape
    d = q.shape[-1] // heads
    q = q.view(b, t, heads, d).transpose(1, 2)
    k = k.view(b, t, kv_heads, d).transpose(1, 2)
    v = v.view(b, t, kv_heads, d).transpose(1, 2)
    c, s = cos[:, None], sin[:, None]
    q, k = q * c + rotate_half(q) * s, k * c + rotate_half(k) * s
    rep = heads // kv_heads
    return (q.half(), k.repeat_interleave(rep, dim=1).half(), v.repeat_interleave(rep, dim=1).half())


@pytest.mark.parametrize("padded", [False, True])
@pytest.mark.parametrize("lengths,seq", [([64, 37, 50, 12], 64), ([334, 200, 100, 7], 334)])
def test_qkv_rotate_matches_transformers(cuda_lib, lengths, seq, padded):
    from hackaton_b200.rope import qkv_rotate

    torch.manual_seed(0)
    batch, heads, kv_heads, dim = len(lengths), 12, 2, 128
    rows, b_idx, t_idx = token_maps(lengths, seq)
    n = rows.numel()
    q = torch.randn(n, heads * dim, device="cuda", requires_grad=True)
    k = torch.randn(n, kv_heads * dim, device="cuda", requires_grad=True)
    v = torch.randn(n, kv_heads * dim, device="cuda", requires_grad=True)
    inv_freq = 1.0 / (1000000.0 ** (torch.arange(0, dim, 2, device="cuda").float() / dim))
    freqs = torch.arange(seq, device="cuda").float()[:, None] * inv_freq[None]
    emb = torch.cat((freqs, freqs), dim=-1)
    cos, sin = emb.cos()[None], emb.sin()[None]
    grads = [torch.randn(batch, heads, seq, dim, device="cuda").half() for _ in range(3)]

    def to_padded(x):
        full = torch.zeros(batch * seq, x.shape[-1], device="cuda")
        return full.index_copy(0, rows, x).view(batch, seq, -1)

    ref = transformers_path(to_padded(q), to_padded(k), to_padded(v), cos.expand(batch, seq, dim),
                            sin.expand(batch, seq, dim), heads, kv_heads)
    torch.autograd.backward(ref, grads)
    ref_grads = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None

    def packed(x):
        return x.transpose(1, 2).reshape(batch * seq, heads, dim)[rows]

    out = qkv_rotate(q, k, v, cos, sin, b_idx, t_idx, batch, seq, heads, kv_heads, padded)
    if padded:
        torch.autograd.backward(out, grads)
        # padding positions of the reference hold rotated zeros = zeros, like ours
    else:
        ref = [packed(x) for x in ref]
        torch.autograd.backward(out, [packed(g) for g in grads])
    for mine, theirs in zip(out, ref):
        torch.testing.assert_close(mine.float(), theirs.float(), rtol=2e-3, atol=2e-3)
    for mine, theirs in zip((q.grad, k.grad, v.grad), ref_grads):
        torch.testing.assert_close(mine, theirs, rtol=2e-3, atol=2e-2)
    # oracle, forward, on the same inputs
    o = nf4_oracle.qkv_rotate_fwd(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), cos.cpu(), sin.cpu(),
                                  b_idx.cpu(), t_idx.cpu(), batch, seq, heads, kv_heads, padded)
    for mine, theirs in zip(out, o):
        torch.testing.assert_close(mine.detach().cpu().float(), theirs.float(), rtol=1e-3, atol=1e-3)
    cuda_lib.device_status()


@pytest.mark.parametrize("heads,kv_heads", [(12, 2), (28, 4), (4, 2), (6, 2)])   # 6, 7, 2 and 3 copies
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_backward_heads_of_128_vs_oracle(cuda_lib, heads, kv_heads, dtype):
    """Packed layout, heads of 128 (the model's head size), several copy counts, both projection
    types: the backward against the oracle on the same gradients."""
    from hackaton_b200.rope import qkv_rotate

    g = torch.Generator().manual_seed(heads * 10 + kv_heads)
    lengths, seq, dim = [9, 4, 7], 9, 128
    b_idx = torch.tensor([b for b, n in enumerate(lengths) for _ in range(n)], dtype=torch.int32)
    t_idx = torch.tensor([t for n in lengths for t in range(n)], dtype=torch.int32)
    n = b_idx.numel()
    q = torch.randn(n, heads * dim, generator=g).to(dtype)
    k = torch.randn(n, kv_heads * dim, generator=g).to(dtype)
    v = torch.randn(n, kv_heads * dim, generator=g).to(dtype)
    ang = torch.arange(seq).float()[:, None] * (1.0 / (1e6 ** (torch.arange(0, dim, 2).float() / dim)))[None]
    cos = torch.cat((ang, ang), -1).cos()[None].contiguous()
    sin = torch.cat((ang, ang), -1).sin()[None].contiguous()
    grads = [torch.randn(n, heads, dim, generator=g).half() for _ in range(3)]
    qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
    outs = qkv_rotate(qg, kg, vg, cos.cuda(), sin.cuda(), b_idx.cuda(), t_idx.cuda(), len(lengths), seq,
                      heads, kv_heads)
    torch.autograd.backward(outs, [x.cuda() for x in grads])
    want = nf4_oracle.qkv_rotate_bwd(*grads, cos, sin, b_idx, t_idx, heads, kv_heads, False, dtype)
    tol = dict(rtol=2e-3, atol=2e-3) if dtype == torch.float16 else dict(rtol=1e-5, atol=1e-5)
    for got, ref in zip((qg.grad, kg.grad, vg.grad), want):
        assert got.dtype == dtype
        torch.testing.assert_close(got.cpu().float(), ref.float(), **tol)
    cuda_lib.device_status()
