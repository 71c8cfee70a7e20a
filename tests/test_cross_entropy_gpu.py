"""GPU: cross-entropy statistics / gradient kernels and the chunked lm_head + loss through the
C ABI against the reference kernel's golden vectors, the oracle and plain PyTorch."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import nf4_oracle

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["ragged", "blocks"])    # 9,001 logits: scalar path; 4,096: vectors
@pytest.mark.parametrize("tag", ["f16", "f32"])
def test_matches_reference_kernel(cuda_lib, name, tag):
    from hackaton_b200.lm_loss import ce_grad, ce_stats

    z = np.load(GOLDEN / "ce_small.npz")
    t = lambda key: torch.from_numpy(z[f"{name}_{tag}_{key}"])
    logits, targets = t("logits").cuda(), torch.from_numpy(z[f"{name}_targets"]).cuda()
    rows = logits.shape[0]
    out = (torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda"),
           torch.empty(rows, dtype=torch.int64, device="cuda"))
    lse, loss, entropy = ce_stats(logits, targets, True, out=out)
    torch.testing.assert_close(lse.cpu(), t("lse"), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(loss.cpu(), t("loss"), rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(entropy.cpu(), t("entropy"), rtol=1e-4, atol=1e-4)
    assert torch.equal(out[3].cpu(), t("argmax"))
    assert float(lse[2]) == 0.0 and float(loss[2]) == 0.0
    scale = torch.tensor([0.37], device="cuda")
    grad = torch.empty_like(logits)
    ce_grad(logits, targets, lse, scale, grad)
    tol = dict(rtol=2e-3, atol=1e-6) if tag == "f16" else dict(rtol=1e-4, atol=1e-7)
    torch.testing.assert_close(grad.cpu().float(), t("grad").float(), **tol)
    assert not bool(grad[2].any())
    work = logits.clone()
    ce_grad(work, targets, lse, scale, work)                   # in place: the same bits
    assert torch.equal(work, grad)
    cuda_lib.device_status()


@pytest.mark.parametrize("rows,vocab,dtype", [(64, 151936, torch.float16), (33, 32000, torch.float32),
                                              (5, 1001, torch.float16)])
def test_fused_cross_entropy_matches_pytorch(cuda_lib, rows, vocab, dtype):
    from hackaton_b200.lm_loss import ce_stats, fused_cross_entropy

    g = torch.Generator(device="cuda").manual_seed(rows + vocab)
    logits = (torch.randn(rows, vocab, device="cuda", generator=g) * 4).to(dtype).requires_grad_()
    targets = torch.randint(0, vocab, (rows,), device="cuda", generator=g)
    targets[1] = -100
    denom = (targets >= 0).sum().float()
    ref = torch.nn.functional.cross_entropy(logits.float(), targets, ignore_index=-100, reduction="sum") / denom
    ref.backward()
    ref_grad = logits.grad.clone()
    logits.grad = None
    loss = fused_cross_entropy(logits, targets, denom)
    loss.backward()
    torch.testing.assert_close(loss, ref, rtol=1e-5, atol=1e-5)
    tol = dict(rtol=2e-3, atol=1e-6) if dtype == torch.float16 else dict(rtol=1e-4, atol=1e-8)
    torch.testing.assert_close(logits.grad.float(), ref_grad.float(), **tol)
    # statistics against the oracle on the same logits
    lse, losses, entropy = ce_stats(logits.detach(), targets, True)
    o_lse, o_loss, o_ent, o_arg = nf4_oracle.ce_stats(logits.detach().cpu(), targets.cpu())
    torch.testing.assert_close(lse.cpu(), o_lse, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(losses.cpu(), o_loss, rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(entropy.cpu(), o_ent, rtol=1e-4, atol=1e-4)
    cuda_lib.device_status()


def test_linear_cross_entropy_matches_unchunked(cuda_lib):
    """solution/lm_loss.py: the chunked lm_head + loss gives the loss, metrics and d loss / d hidden
    of the plain computation (600 rows = three chunks, the last one ragged)."""
    from hackaton_b200.lm_loss import linear_cross_entropy

    g = torch.Generator(device="cuda").manual_seed(11)
    rows, hidden_size, vocab = 600, 256, 5000
    hidden = (torch.randn(rows, hidden_size, device="cuda", generator=g) * 0.5).half().requires_grad_()
    weight = (torch.randn(vocab, hidden_size, device="cuda", generator=g) * 0.1).half()
    targets = torch.randint(0, vocab, (rows,), device="cuda", generator=g)
    targets[::7] = -100
    denom = (targets >= 0).sum().float()
    logits = torch.nn.functional.linear(hidden, weight)
    ref = torch.nn.functional.cross_entropy(logits.float(), targets, ignore_index=-100, reduction="sum") / denom
    ref.backward()
    ref_grad = hidden.grad.clone()
    hidden.grad = None
    loss, losses, entropy, argmax = linear_cross_entropy(hidden, weight, targets, denom)
    loss.backward()
    torch.testing.assert_close(loss, ref, rtol=1e-4, atol=1e-4)
    assert torch.equal(argmax, torch.argmax(logits.float(), dim=-1))
    o = nf4_oracle.ce_stats(logits.detach().cpu(), targets.cpu())
    torch.testing.assert_close(losses.cpu(), o[1], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(entropy.cpu(), o[2], rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(hidden.grad.float(), ref_grad.float(), rtol=2e-2, atol=2e-6)
    cuda_lib.device_status()
