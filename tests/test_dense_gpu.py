"""GPU: the fp16-weight linear (`fp16_linear`, the lm_head products of the chunked loss) through
the C ABI against a plain PyTorch fp32 product of the same operands; tolerance: max |err| /
max |ref| <= 2e-3 (fp16 output rounding plus fp32 summation order)."""

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _rel(got, want):
    return float((got.float() - want).abs().max() / want.abs().max())


# (M, N, K): single-CTA, 256-row and 512-row tile plans, ragged edges, one contraction block
CASES = [(1, 264, 64), (100, 1000, 320), (256, 1536, 1536), (300, 512, 1536), (700, 264, 320),
         (2048, 1536, 1536), (33, 4096, 128)]


@pytest.mark.parametrize("m,n,k", CASES)
def test_fp16_linear_both_directions(cuda_lib, m, n, k):
    from hackaton_b200 import fp16_linear

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    w = (torch.randn(n, k, generator=g, device="cuda") * 0.05).half()
    x = torch.randn(m, k, generator=g, device="cuda").half()
    dy = torch.randn(m, n, generator=g, device="cuda").half()
    bias = torch.randn(n, generator=g, device="cuda").half()
    y = fp16_linear(x, w, bias=bias)
    assert _rel(y, x.float() @ w.float().t() + bias.float()) <= TOL
    dx = fp16_linear(dy, w, transposed=True)
    assert _rel(dx, dy.float() @ w.float()) <= TOL
    assert cuda_lib.device_status() == 0


def test_fp16_linear_padded_rows_and_out_argument(cuda_lib):
    """Weight, input and output with row strides larger than their widths; `out` is filled in place."""
    from hackaton_b200 import fp16_linear

    g = torch.Generator(device="cuda").manual_seed(5)
    w_full = (torch.randn(512, 320, generator=g, device="cuda") * 0.05).half()
    w = w_full[:, :256]                       # row stride 320
    x = torch.randn(3, 40, 384, generator=g, device="cuda").half()[..., :256]
    y = fp16_linear(x, w)
    assert y.shape == (3, 40, 512)
    assert _rel(y.reshape(-1, 512), x.reshape(-1, 256).float() @ w.float().t()) <= TOL
    buf = torch.zeros(120, 264, dtype=torch.float16, device="cuda")
    out = buf[:, :256]
    dy = torch.randn(120, 512, generator=g, device="cuda").half()
    fp16_linear(dy, w, transposed=True, out=out)
    assert _rel(out, dy.float() @ w.float()) <= TOL
    assert float(buf[:, 256:].abs().max()) == 0.0
    with pytest.raises(TypeError):
        fp16_linear(x.float(), w)


def test_lm_head_chunk_at_the_real_vocabulary(cuda_lib):
    """One chunk of the chunked loss at Qwen2.5-1.5B's sizes: 256 rows against the 151,936 x 1536
    table, logits and the product back to the hidden size (a contraction over 151,936)."""
    from hackaton_b200 import fp16_linear

    g = torch.Generator(device="cuda").manual_seed(9)
    vocab, hidden, rows = 151936, 1536, 256
    w = (torch.randn(vocab, hidden, generator=g, device="cuda") * 0.02).half()
    h = torch.randn(rows, hidden, generator=g, device="cuda").half()
    logits = fp16_linear(h, w)
    assert _rel(logits, h.float() @ w.float().t()) <= TOL
    d_logits = (torch.randn(rows, vocab, generator=g, device="cuda") * 0.01).half()
    d_hidden = fp16_linear(d_logits, w, transposed=True)
    assert _rel(d_hidden, d_logits.float() @ w.float()) <= TOL
    assert cuda_lib.device_status() == 0
