"""GPU: the device status word. A kernel that meets something it must report (a bounded wait that
ran out, a label beyond the vocabulary, a block scale fp16 cannot hold) records a code and ends
normally; `nf4b200_device_status` then returns NF4B200_EDEVICE once and the context stays usable.
None of these cases faults, traps or hangs the GPU: the waiting kernel gives up after a
millisecond by itself, and the out-of-range accesses are skipped, not performed."""

import ctypes

import pytest
import torch

from oracle import nf4_oracle
from tests.util import oracle_weight, synthetic_weight

pytestmark = pytest.mark.gpu


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _works_afterwards(cuda_lib):
    from hackaton_b200.nf4 import linear_forward

    packed, state = synthetic_weight(256, 128, True, seed=1, device="cuda")
    x = torch.randn(40, 128).half()
    y = linear_forward(x.cuda(), packed, None, state)
    assert nf4_oracle.max_rel_err(y.cpu(), nf4_oracle.linear_fwd(x, oracle_weight(packed, state))) <= 1e-2
    assert cuda_lib.device_status() == 0


def test_bounded_wait_runs_out_and_is_reported(cuda_lib):
    assert cuda_lib.device_status() == 0
    cuda_lib.check(cuda_lib.lib().nf4b200_selftest_wait(1_000_000, _stream()))   # 1 ms
    with pytest.raises(cuda_lib.Nf4Error) as info:
        cuda_lib.device_status()
    assert info.value.code == -4 and "400" in str(info.value)
    assert cuda_lib.device_status() == 0          # reading the word cleared it
    with pytest.raises(cuda_lib.Nf4Error):        # limits beyond one second are refused on the host
        cuda_lib.check(cuda_lib.lib().nf4b200_selftest_wait(5_000_000_000, _stream()))
    _works_afterwards(cuda_lib)


def test_label_beyond_the_vocabulary_is_an_ignored_row(cuda_lib):
    from hackaton_b200.lm_loss import ce_grad, ce_stats

    vocab = 1000
    g = torch.Generator().manual_seed(0)
    logits = (torch.randn(5, vocab, generator=g) * 2).half()
    targets = torch.tensor([5, vocab, 2_000_000_000, -100, 999])
    lse, loss, _ = ce_stats(logits.cuda(), targets.cuda(), False)
    grad = torch.empty(5, vocab, dtype=torch.float16, device="cuda")
    ce_grad(logits.cuda(), targets.cuda(), lse, torch.ones(1, device="cuda"), grad)
    with pytest.raises(cuda_lib.Nf4Error) as info:
        cuda_lib.device_status()
    assert "200" in str(info.value)
    ok = torch.tensor([True, False, False, False, True])
    want = nf4_oracle.ce_stats(logits, torch.where(ok, targets, torch.full_like(targets, -100)))[1]
    torch.testing.assert_close(loss.cpu(), want, rtol=1e-4, atol=1e-4)
    assert float(loss[1]) == 0.0 and float(loss[2]) == 0.0 and float(loss[3]) == 0.0
    assert float(grad[1:4].float().abs().max()) == 0.0
    assert float(grad[0].float().abs().max()) > 0.0
    _works_afterwards(cuda_lib)


def test_block_scale_outside_fp16_range_is_reported(cuda_lib):
    from hackaton_b200.nf4 import dequantize_nf4, weight_ref

    packed, state = synthetic_weight(64, 128, False, seed=2, device="cuda")   # flat fp32 scales
    state.absmax = state.absmax.clone()
    state.absmax[3] = 1e-7          # fp16 would make this a subnormal
    w = dequantize_nf4(packed, state)      # the standalone decode multiplies in fp32: exact
    assert torch.equal(w.cpu(), oracle_weight(packed, state))
    assert cuda_lib.device_status() == 0
    weight_ref(packed.reshape(-1), state).prepare()
    with pytest.raises(cuda_lib.Nf4Error) as info:
        cuda_lib.device_status()
    assert "300" in str(info.value)
    _works_afterwards(cuda_lib)
