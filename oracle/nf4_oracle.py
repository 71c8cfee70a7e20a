"""Plain numpy / torch-CPU restatement of the reference's NF4 hot path (test infrastructure).

Every function names the reference lines it follows. Parity status is stated in the package
docstring (oracle/__init__.py): the flat decode and the linear are pinned by golden vectors made
with the reference's own code; the nested-absmax decode and LoRA are "parity unpinned". The
steps either side of the projections (SwiGLU, RMSNorm, q/k/v rotation + grouped-query expansion,
cross-entropy) are restated at the end of this file and pinned the same way, by golden vectors of
the reference's own kernels (tests/golden/make_golden_*.py).

Byte and nibble layout (solution/nf4.py:7-14, 33-44): flat element i of the row-major weight sits
in byte i // 2; the even element is the HIGH nibble, the odd one the LOW nibble; `blocksize`
consecutive flat elements share one scale. value = table[code] * scale in fp32, rounded once to
the output dtype.
"""

from __future__ import annotations

import numpy as np
import torch


# --------------------------------------------------------------------------------------------
# decode
# --------------------------------------------------------------------------------------------

def flatten_absmax(absmax_u8, code2, absmax2, offset, nested_blocksize=256):
    """Two-level scales -> flat fp32 scales.

    Follows solution/packed.py:74-77 and solution/test_nf4.py:23-26: a blockwise 8-bit decode
    (`code2[u8] * absmax2[i // nested_blocksize]`, one fp32 multiply) followed by an in-place
    fp32 `+= offset` (a second, separately rounded fp32 op; never a fused multiply-add).
    """
    absmax_u8 = np.asarray(absmax_u8, dtype=np.uint8).reshape(-1)
    code2 = np.asarray(code2, dtype=np.float32).reshape(-1)
    absmax2 = np.asarray(absmax2, dtype=np.float32).reshape(-1)
    idx = np.arange(absmax_u8.size, dtype=np.int64) // nested_blocksize
    prod = (code2[absmax_u8] * absmax2[idx]).astype(np.float32)
    return (prod + np.float32(offset)).astype(np.float32)


def nibbles(packed):
    """Packed bytes -> 4-bit codes in flat element order (high nibble first, nf4.py:8,34,40)."""
    packed = np.asarray(packed, dtype=np.uint8).reshape(-1)
    out = np.empty(packed.size * 2, dtype=np.uint8)
    out[0::2] = packed >> 4
    out[1::2] = packed & 15
    return out


def dequant_flat(packed, absmax_f32, code16, shape, blocksize=64, dtype=torch.float16):
    """Decode with flat fp32 scales: solution/nf4.py:33-44 (one fp32 multiply, one rounding).

    Returns a torch CPU tensor of `shape` and `dtype` (fp16, bf16 or fp32).
    """
    n = int(np.prod(shape))
    codes = nibbles(packed)[:n]
    table = np.asarray(code16, dtype=np.float32).reshape(-1)
    scale = np.asarray(absmax_f32, dtype=np.float32).reshape(-1)
    block = np.arange(n, dtype=np.int64) // blocksize
    value = (table[codes] * scale[block]).astype(np.float32)
    out = torch.from_numpy(value).to(dtype)  # round-to-nearest-even, one rounding
    return out.reshape(tuple(shape))


def dequant_nested(packed, absmax_u8, code2, absmax2, offset, code16, shape, blocksize=64,
                   nested_blocksize=256, dtype=torch.float16):
    """Double-quantised layout decoded in one go: flatten_absmax, then dequant_flat."""
    flat = flatten_absmax(absmax_u8, code2, absmax2, offset, nested_blocksize)
    return dequant_flat(packed, flat, code16, shape, blocksize, dtype)


# --------------------------------------------------------------------------------------------
# linear (solution/nf4.py:80-102) and LoRA (peft's `Linear.forward`, configured at
# README.md:91 / task/task.yaml:18-21 of the reference; not in its tree)
# --------------------------------------------------------------------------------------------

def linear_fwd(x, weight, bias=None):
    """Y = X Wᵀ (+ bias), fp32 accumulate, result in x's dtype (nf4.py:87-92)."""
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def linear_bwd(grad_y, weight):
    """dX = dY W, fp32 accumulate (nf4.py:94-99)."""
    return (grad_y.float() @ weight.float()).to(grad_y.dtype)


def bias_grad(grad_y, dtype):
    """dbias = dY summed over rows (nf4.py:100-101)."""
    return grad_y.reshape(-1, grad_y.shape[-1]).float().sum(0).to(dtype)


def lora_fwd(x, weight, lora_a, lora_b, scaling, bias=None):
    """Y = X Wᵀ (+ bias) + scaling * (X Aᵀ) Bᵀ with the low-rank product kept in fp32.

    A is [r, K], B is [N, r]. Returns (Y, XA) where XA = X Aᵀ in fp32 (the tensor a fused kernel
    hands to the backward pass).
    """
    xa = x.float() @ lora_a.float().t()
    y = x.float() @ weight.float().t() + scaling * (xa @ lora_b.float().t())
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype), xa


def lora_bwd(grad_y, x, weight, lora_a, lora_b, scaling):
    """Gradients of lora_fwd w.r.t. X, A and B (W frozen), fp32 accumulate.

    dX = dY W + scaling * (dY B) A;  dA = scaling * (dY B)ᵀ X;  dB = scaling * dYᵀ (X Aᵀ).
    """
    gy, xf = grad_y.float(), x.float()
    a, b = lora_a.float(), lora_b.float()
    gyb = gy @ b                                  # [M, r]
    dx = gy @ weight.float() + scaling * (gyb @ a)
    da = scaling * (gyb.t() @ xf)                 # [r, K]
    db = scaling * (gy.t() @ (xf @ a.t()))        # [N, r]
    return dx.to(grad_y.dtype), da, db


def swiglu_fwd(gate, up):
    """hidden = silu(gate) * up as the reference's `silu_mul_kernel` forms it, mode 0
    (solution/kernels.py:43-47): fp16 values widened to fp32, `gate * sigmoid(gate) * up`, one
    rounding to the output type."""
    g, u = gate.detach().float(), up.detach().float()
    return (g * torch.sigmoid(g) * u).to(gate.dtype)


def swiglu_bwd(d_hidden, gate, up):
    """(d_gate, d_up), mode 1 of the same kernel (solution/kernels.py:48-57):
    d_up = dout * gate * sig; d_gate = (dout * up) * sig * (1 + gate * (1 - sig))."""
    d, g, u = d_hidden.detach().float(), gate.detach().float(), up.detach().float()
    sig = torch.sigmoid(g)
    d_up = d * g * sig
    d_gate = (d * u) * sig * (1.0 + g * (1.0 - sig))
    return d_gate.to(gate.dtype), d_up.to(up.dtype)


def rmsnorm_fwd(x, weight, eps, delta=None, out_dtype=torch.float32):
    """Modes 0 and 2 of the reference's rmsnorm_kernel (solution/rmsnorm.py:27-36): s = x (+ delta,
    widened to fp32), rstd = 1 / sqrt(sum(s^2) / hidden + eps), y = w * (s * rstd) rounded to
    `out_dtype`. Returns (y, rstd, s)."""
    s = x.detach().float()
    if delta is not None:
        s = s + delta.detach().float()
    rstd = 1.0 / torch.sqrt((s * s).sum(dim=-1) / s.shape[-1] + eps)
    y = weight.detach().float() * (s * rstd[..., None])
    return y.to(out_dtype), rstd, s


def rmsnorm_bwd(x, weight, rstd, dy, d_total=None):
    """Modes 1 and 3 (solution/rmsnorm.py:37-48): xhat = x * rstd, g = dy * w,
    dx = rstd * (g - xhat * sum(g * xhat) / hidden) (+ d_total)."""
    xhat = x.detach().float() * rstd[..., None]
    g = dy.detach().float() * weight.detach().float()
    mean_gx = (g * xhat).sum(dim=-1, keepdim=True) / x.shape[-1]
    dx = rstd[..., None] * (g - xhat * mean_gx)
    if d_total is not None:
        dx = dx + d_total.detach().float()
    return dx


def _rope_rows(cos, sin, b_idx, t_idx):
    """cos / sin rows of each packed token: (1 or B, T, D) indexed by (b, t) (solution/attention.py:45-49)."""
    b = b_idx.long() if cos.shape[0] > 1 else torch.zeros_like(b_idx.long())
    return cos[b, t_idx.long()].float(), sin[b, t_idx.long()].float()


def qkv_rotate_fwd(q, k, v, cos, sin, b_idx, t_idx, batch, seq, heads, kv_heads, padded):
    """The reference's `_qkv_forward` (solution/attention.py:36-83): per head, over its two halves,
    y1 = x1*c1 - x2*s1, y2 = x2*c2 + x1*s2 in fp32, rounded to fp16; k and v heads repeated
    heads / kv_heads times; rows packed (N, H, D) or scattered into zeros (B, H, T, D)."""
    n, dim = q.shape[0], q.shape[-1] // heads
    half, rep = dim // 2, heads // kv_heads
    c, s = _rope_rows(cos, sin, b_idx, t_idx)
    c1, c2, s1, s2 = c[:, None, :half], c[:, None, half:], s[:, None, :half], s[:, None, half:]

    def rotate(x, nh):
        x = x.detach().float().reshape(n, nh, dim)
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat((x1 * c1 - x2 * s1, x2 * c2 + x1 * s2), dim=-1).half()

    qo = rotate(q, heads)
    ko = rotate(k, kv_heads).repeat_interleave(rep, dim=1)
    vo = v.detach().reshape(n, kv_heads, dim).half().repeat_interleave(rep, dim=1)
    if not padded:
        return qo, ko, vo
    outs = []
    for x in (qo, ko, vo):
        full = torch.zeros(batch, heads, seq, dim, dtype=torch.float16)
        full[b_idx.long(), :, t_idx.long()] = x
        outs.append(full)
    return tuple(outs)


def qkv_rotate_bwd(dq, dk, dv, cos, sin, b_idx, t_idx, heads, kv_heads, padded, dtype):
    """The reference's `_qkv_backward` (solution/attention.py:86-133): the copies' gradients summed
    in fp32, dx1 = dy1*c1 + dy2*s2, dx2 = dy2*c2 - dy1*s1, written (N, heads * D) in `dtype`."""
    if padded:
        dq, dk, dv = (g[b_idx.long(), :, t_idx.long()] for g in (dq, dk, dv))
    n, dim = dq.shape[0], dq.shape[-1]
    half, rep = dim // 2, heads // kv_heads
    c, s = _rope_rows(cos, sin, b_idx, t_idx)
    c1, c2, s1, s2 = c[:, None, :half], c[:, None, half:], s[:, None, :half], s[:, None, half:]

    def unrotate(d):
        d1, d2 = d[..., :half], d[..., half:]
        return torch.cat((d1 * c1 + d2 * s2, d2 * c2 - d1 * s1), dim=-1)

    dq = unrotate(dq.float()).reshape(n, heads * dim)
    dk = unrotate(dk.float().reshape(n, kv_heads, rep, dim).sum(dim=2)).reshape(n, kv_heads * dim)
    dv = dv.float().reshape(n, kv_heads, rep, dim).sum(dim=2).reshape(n, kv_heads * dim)
    return dq.to(dtype), dk.to(dtype), dv.to(dtype)


def ce_stats(logits, targets):
    """The statistics pass of the reference's ce_kernel (solution/kernels.py:106-146), per row of
    logits (here in float64, rounded to fp32 at the end): lse = logsumexp (0 for target < 0), loss = lse - logit[target] (0 for
    those rows), entropy = lse - E_softmax[x], argmax = first maximal index."""
    x = logits.detach().double()        # float64: the sums run over 10^5 terms
    lse = torch.logsumexp(x, dim=-1)
    p = torch.softmax(x, dim=-1)
    entropy = lse - (p * x).sum(dim=-1)
    argmax = torch.argmax(x, dim=-1)                    # torch returns the first maximum
    valid = targets >= 0
    picked = x.gather(1, targets.clamp_min(0)[:, None])[:, 0]
    zero = torch.zeros_like(lse)
    return (torch.where(valid, lse, zero).float(), torch.where(valid, lse - picked, zero).float(),
            entropy.float(), argmax)


def ce_grad(logits, targets, lse, scale):
    """The gradient pass (solution/kernels.py:149-165): scale * (exp(x - lse) - onehot(target)),
    0 for rows with target < 0, rounded to the logits' type."""
    x = logits.detach().float()
    g = torch.exp(x - lse[:, None])
    valid = targets >= 0
    g[torch.arange(x.shape[0])[valid], targets[valid]] -= 1.0
    g = g * float(scale)
    g[~valid] = 0.0
    return g.to(logits.dtype)


def max_rel_err(got, want):
    """max |got - want| / max |want| : the error measure of the fp16 tolerance (<= 1e-2)."""
    got, want = got.detach().float(), want.detach().float()
    denom = want.abs().max().clamp_min(1e-30)
    return float((got - want).abs().max() / denom)


# --------------------------------------------------------------------------------------------
# threaded variant for the timed CPU baseline
# --------------------------------------------------------------------------------------------

def dequant_torch(packed, absmax, code16, shape, blocksize=64, dtype=torch.float16, code2=None,
                  absmax2=None, offset=None, nested_blocksize=256):
    """Same arithmetic as dequant_flat / dequant_nested written with torch CPU ops, so that it
    uses all host threads: the reference's plain-PyTorch decode path timed as the CPU baseline
    (its decode, solution/nf4.py:33-44, followed by F.linear / matmul, :87-99)."""
    packed = torch.as_tensor(packed).reshape(-1)
    n = 1
    for d in shape:
        n *= int(d)
    table = torch.as_tensor(code16, dtype=torch.float32)
    if code2 is not None:
        q = torch.as_tensor(absmax).reshape(-1).long()
        idx = torch.arange(q.numel()) // nested_blocksize
        scale = torch.as_tensor(code2, dtype=torch.float32)[q] * \
            torch.as_tensor(absmax2, dtype=torch.float32)[idx]
        scale = scale + torch.as_tensor(offset, dtype=torch.float32)
    else:
        scale = torch.as_tensor(absmax, dtype=torch.float32).reshape(-1)
    hi = table[(packed >> 4).long()]
    lo = table[(packed & 15).long()]
    value = torch.stack((hi, lo), dim=1).reshape(-1)[:n]
    value = (value.view(-1, blocksize) * scale[:, None]).reshape(-1)
    return value.to(dtype).reshape(tuple(shape))
