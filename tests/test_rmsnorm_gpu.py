"""GPU: RMSNorm and add + RMSNorm through the C ABI against the reference kernel's golden
vectors, the oracle and plain PyTorch (the reference's own tests, solution/test_norm_and_stats.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import nf4_oracle

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["qwen", "odd"])      # 1536: register-resident kernel; 1000: generic
@pytest.mark.parametrize("tag", ["f32", "f16"])
def test_matches_reference_kernel(cuda_lib, name, tag):
    from hackaton_b200.rmsnorm import launch_backward as _backward, launch_forward as _forward

    z = np.load(GOLDEN / "rmsnorm_small.npz")
    t = lambda key: torch.from_numpy(z[f"{name}_{key}"])
    half = tag == "f16"
    x, w, delta, d_total = (t(k).cuda() for k in ("x", "w", "delta", "d_total"))
    dy = t("dy").to(torch.float16 if half else torch.float32).cuda()
    tol = dict(rtol=1e-3, atol=1e-3) if half else dict(rtol=2e-6, atol=2e-6)
    y, rstd, _ = _forward(x, None, w, 1e-6, half)
    torch.testing.assert_close(y.cpu().float(), t(f"{tag}_y").float(), **tol)
    torch.testing.assert_close(rstd.cpu(), t(f"{tag}_rstd"), rtol=2e-6, atol=0)
    dx = _backward(x, w, rstd, dy, None)
    torch.testing.assert_close(dx.cpu(), t(f"{tag}_dx"), rtol=2e-5, atol=2e-6)
    y2, rstd2, total = _forward(x, delta, w, 1e-6, half)
    assert torch.equal(total.cpu(), t(f"{tag}_total"))
    torch.testing.assert_close(y2.cpu().float(), t(f"{tag}_y_add").float(), **tol)
    dx2 = _backward(total, w, rstd2, dy, d_total)
    torch.testing.assert_close(dx2.cpu(), t(f"{tag}_dx_add"), rtol=2e-5, atol=2e-6)
    cuda_lib.device_status()


@pytest.mark.parametrize("shape", [(4, 334, 1536), (3, 77, 1000), (2, 50, 3584)])
@pytest.mark.parametrize("train_weight", [False, True])
@pytest.mark.parametrize("to_half", [False, True])
def test_rms_norm_matches_qwen2(cuda_lib, shape, train_weight, to_half):
    """solution/test_norm_and_stats.py:9-39, same tolerances (plus the 7B width)."""
    from hackaton_b200.rmsnorm import rms_norm

    torch.manual_seed(0)
    x = torch.randn(shape, device="cuda", requires_grad=True)
    weight = (1 + 0.1 * torch.randn(shape[-1], device="cuda")).requires_grad_(train_weight)
    dy = torch.randn(shape, device="cuda")
    eps = 1e-6
    out_dtype = torch.float16 if to_half else torch.float32
    variance = x.pow(2).mean(-1, keepdim=True)
    ref = (weight * (x * torch.rsqrt(variance + eps))).to(out_dtype)
    ref.backward(dy.to(out_dtype))
    ref_dx = x.grad.clone()
    ref_dw = weight.grad.clone() if train_weight else None
    x.grad = None
    if train_weight:
        weight.grad = None
    out = rms_norm(x, weight, eps, to_half)
    assert out.dtype == out_dtype
    out.backward(dy.to(out_dtype))
    tol = 2e-3 if to_half else 1e-5
    torch.testing.assert_close(out.float(), ref.float(), rtol=tol, atol=tol)
    torch.testing.assert_close(x.grad, ref_dx, rtol=1e-3 if to_half else 1e-4, atol=1e-3 if to_half else 1e-5)
    if train_weight:
        torch.testing.assert_close(weight.grad, ref_dw, rtol=2e-3 if to_half else 1e-4,
                                   atol=3e-2 if to_half else 1e-3)
    # and the oracle, forward
    y_o, _, _ = nf4_oracle.rmsnorm_fwd(x.detach().cpu(), weight.detach().cpu(), eps, None, out_dtype)
    torch.testing.assert_close(out.detach().cpu().float(), y_o.float(), rtol=tol, atol=tol)
    cuda_lib.device_status()


@pytest.mark.parametrize("train_weight", [False, True])
@pytest.mark.parametrize("to_half", [True, False])
def test_add_rmsnorm_matches_add_then_rmsnorm(cuda_lib, to_half, train_weight):
    """solution/test_norm_and_stats.py:75-102."""
    from hackaton_b200.rmsnorm import add_rms_norm, rms_norm

    torch.manual_seed(0)
    residual = torch.randn(300, 1536, device="cuda", requires_grad=True)
    delta = torch.randn(300, 1536, device="cuda").half().requires_grad_()
    weight = (torch.rand(1536, device="cuda") + 0.5).requires_grad_(train_weight)
    g_total = torch.randn(300, 1536, device="cuda")
    g_out = torch.randn(300, 1536, device="cuda")
    total = residual + delta
    out = rms_norm(total, weight, 1e-6, to_half=to_half)
    torch.autograd.backward([total, out], [g_total, g_out.to(out.dtype)])
    ref = [total.detach(), out.detach(), residual.grad.clone(), delta.grad.clone()]
    ref_w = weight.grad.clone() if train_weight else None
    residual.grad = delta.grad = weight.grad = None
    total, out = add_rms_norm(residual, delta, weight, 1e-6, to_half=to_half)
    torch.autograd.backward([total, out], [g_total, g_out.to(out.dtype)])
    mine = [total.detach(), out.detach(), residual.grad, delta.grad]
    if train_weight:
        torch.testing.assert_close(weight.grad, ref_w, rtol=1e-3, atol=1e-2)
    assert torch.equal(mine[0], ref[0])  # the sum is the same fp32 addition
    for a, b in zip(mine[1:], ref[1:]):
        assert a.dtype == b.dtype
        torch.testing.assert_close(a.float(), b.float(), rtol=1e-3, atol=1e-3)
    cuda_lib.device_status()


def test_empty_and_errors(cuda_lib):
    from hackaton_b200.rmsnorm import rms_norm

    w = torch.ones(1536, device="cuda")
    assert rms_norm(torch.empty(0, 1536, device="cuda"), w, 1e-6, True).shape == (0, 1536)
    with pytest.raises(TypeError):
        rms_norm(torch.zeros(2, 1536, device="cuda").half(), w, 1e-6)
    with pytest.raises(ValueError):
        rms_norm(torch.zeros(2, 1024, device="cuda"), w, 1e-6)
