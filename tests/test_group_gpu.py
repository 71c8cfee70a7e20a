"""GPU: grouped launches (q/k/v sharing one input, their input gradients summed) through the C
ABI against the oracle and against the one-projection-at-a-time path."""

import pytest
import torch

from oracle import nf4_oracle
from tests.util import oracle_weight, synthetic_weight

pytestmark = pytest.mark.gpu
TOL = 1e-2


def build(m, k, ns, lora_on, seed):
    from hackaton_b200 import Projection

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).half()
    projs, cpu = [], []
    for i, n in enumerate(ns):
        packed, state = synthetic_weight(n, k, True, seed=seed + i, device="cuda")
        w = oracle_weight(packed, state)
        dy = torch.randn(m, n, generator=g).half()
        bias = (torch.randn(n, generator=g) * 0.1).half() if i == 1 else None
        a = b = None
        if i in lora_on:
            a = ((torch.rand(16, k, generator=g) * 2 - 1) / k ** 0.5).half()
            b = (torch.randn(n, 16, generator=g) * 0.2).half()
        cpu.append((w, dy, bias, a, b))
        projs.append(Projection(packed, state,
                                None if bias is None else bias.cuda().requires_grad_(),
                                None if a is None else a.cuda().requires_grad_(),
                                None if b is None else b.cuda().requires_grad_(), 2.0))
    return x, projs, cpu


@pytest.mark.parametrize("m,k,ns,lora_on", [
    (2048, 1536, (1536, 256, 256), (0, 2)),   # q, k, v of Qwen2.5-1.5B with LoRA on q and v
    (300, 192, (264, 64, 8), (1,)),           # ragged sizes
    (2048, 1536, (512, 512), ()),             # no LoRA
    (64, 128, (256, 256, 128, 64), (3,)),     # single-CTA tiles, four members
])
def test_group_forward_backward_vs_oracle(cuda_lib, m, k, ns, lora_on):
    from hackaton_b200 import nf4_linear_group

    x, projs, cpu = build(m, k, ns, lora_on, seed=m + k)
    xg = x.cuda().requires_grad_()
    ys = nf4_linear_group(xg, projs)
    torch.autograd.backward(list(ys), [c[1].cuda() for c in cpu])
    torch.cuda.synchronize()
    dx_ref = torch.zeros(m, k)
    for y, pr, (w, dy, bias, a, b) in zip(ys, projs, cpu):
        if a is None:
            y_ref = nf4_oracle.linear_fwd(x, w, bias)
            dx_ref += dy.float() @ w.float()
        else:
            y_ref, _ = nf4_oracle.lora_fwd(x, w, a, b, 2.0, bias)
            dxi, da, db = nf4_oracle.lora_bwd(dy, x, w, a, b, 2.0)
            dx_ref += dy.float() @ w.float() + 2.0 * (dy.float() @ b.float()) @ a.float()
            assert nf4_oracle.max_rel_err(pr.lora_a.grad.cpu(), da) <= TOL
            assert nf4_oracle.max_rel_err(pr.lora_b.grad.cpu(), db) <= TOL
        assert nf4_oracle.max_rel_err(y.detach().cpu(), y_ref) <= TOL
        if bias is not None:
            torch.testing.assert_close(pr.bias.grad.float().cpu(), dy.float().sum(0), rtol=2e-2, atol=2e-1)
    assert nf4_oracle.max_rel_err(xg.grad.cpu(), dx_ref) <= TOL
    cuda_lib.device_status()


def test_group_equals_one_at_a_time(cuda_lib):
    from hackaton_b200 import nf4_linear
    from hackaton_b200.group import linear_backward_dx_group, linear_forward_group
    from hackaton_b200.nf4 import linear_backward_dx

    m, k, ns = 2048, 1536, (1536, 256, 256)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(m, k, generator=g, device="cuda").half()
    ws = [synthetic_weight(n, k, True, seed=40 + i, device="cuda") for i, n in enumerate(ns)]
    ys = linear_forward_group(x, ws)
    for y, (packed, state) in zip(ys, ws):
        one = nf4_linear(x, packed, None, state)
        assert float((y.float() - one.float()).abs().max() / one.float().abs().max()) < 2e-3
    dys = [torch.randn(m, n, generator=g, device="cuda").half() for n in ns]
    dx = linear_backward_dx_group(dys, ws)
    ref = sum(linear_backward_dx(dy, p, s).float() for dy, (p, s) in zip(dys, ws))
    assert float((dx.float() - ref).abs().max() / ref.abs().max()) < 5e-3


def test_sibling_modules_share_one_launch(cuda_lib):
    """Module-level grouping: q/k/v-like modules patched with SiblingGroup give the same results
    as calling each projection's own fused op, forward and backward, and LoRA wrappers with
    attributes like peft's are followed."""
    import types

    from hackaton_b200 import nf4_linear, nf4_lora_linear
    from hackaton_b200.patches import SiblingGroup

    m, k, ns = 512, 1536, (1536, 256, 256)
    g = torch.Generator(device="cuda").manual_seed(5)

    class Base(torch.nn.Module):
        def __init__(self, n, seed):
            super().__init__()
            packed, state = synthetic_weight(n, k, True, seed=seed, device="cuda")
            self.weight = packed
            self.weight.quant_state = state
            self.bias = None
            self.in_features = k

        def forward(self, x):
            return nf4_linear(x, self.weight, self.bias, self.weight.quant_state)

    class Wrapped(torch.nn.Module):
        def __init__(self, n, seed):
            super().__init__()
            self.base_layer = Base(n, seed)
            a = ((torch.rand(16, k, generator=g, device="cuda") * 2 - 1) / k ** 0.5).half()
            b = (torch.randn(n, 16, generator=g, device="cuda") * 0.2).half()
            self.lora_A = {"default": types.SimpleNamespace(weight=a.requires_grad_(), bias=None)}
            self.lora_B = {"default": types.SimpleNamespace(weight=b.requires_grad_(), bias=None)}
            self.lora_dropout = {"default": torch.nn.Identity()}
            self.scaling = {"default": 2.0}
            self.active_adapters = ["default"]
            self.disable_adapters = False
            self.merged = False

        def forward(self, x):
            b = self.base_layer
            return nf4_lora_linear(x, b.weight, b.bias, b.weight.quant_state,
                                   self.lora_A["default"].weight, self.lora_B["default"].weight, 2.0)

    mods = [Wrapped(ns[0], 70), Base(ns[1], 71), Wrapped(ns[2], 72)]
    x = torch.randn(m, k, generator=g, device="cuda").half()
    dys = [torch.randn(m, n, generator=g, device="cuda").half() for n in ns]

    def run():
        xg = x.clone().requires_grad_()
        ys = [mod(xg) for mod in mods]
        torch.autograd.backward(ys, dys)
        grads = [xg.grad.clone()]
        for mod in mods:
            if hasattr(mod, "lora_A"):
                for d in (mod.lora_A, mod.lora_B):
                    grads.append(d["default"].weight.grad.clone())
                    d["default"].weight.grad = None
        return [y.detach() for y in ys], grads

    ys_ref, grads_ref = run()
    group = SiblingGroup(mods).install()
    ys, grads = run()
    assert group._shares == {} and group._x is None         # every share was collected
    group.remove()
    for y, r in zip(ys, ys_ref):
        assert nf4_oracle.max_rel_err(y.cpu(), r.cpu()) <= 2e-3
    for a, r in zip(grads, grads_ref):
        assert nf4_oracle.max_rel_err(a.cpu(), r.cpu()) <= 1e-2
    cuda_lib.device_status()


def test_launch_count_query(cuda_lib):
    """nf4b200_launches_group: one GEMM, plus one reduction per output where the plan cuts the
    contraction into K-slices (1.5B shapes at 2048 tokens)."""
    import ctypes

    lib = cuda_lib.lib()

    def launches(rows, cols, m, backward, tables=1):
        arr = (ctypes.c_int64 * len(rows))(*rows)
        return int(lib.nf4b200_launches_group(len(rows), arr, cols, m, backward, tables))

    qkv, gate_up = (1536, 256, 256), (8960, 8960)
    assert launches(qkv, 1536, 2048, 0) == 1          # 512 x 128 tiles, one wave
    assert launches(qkv, 1536, 2048, 1) == 1          # ... also for the chained backward
    assert launches(qkv, 1536, 2048, 1, tables=0) == 2   # without scale tables: K-slices + reduction
    assert launches(gate_up, 1536, 2048, 0) == 1
    assert launches(gate_up, 1536, 2048, 1) == 2      # 280 k-blocks over 24 tiles: three K-slices
    assert launches((1536,), 8960, 2048, 0) == 2      # down forward
    assert launches((1536,), 8960, 2048, 1) == 1
    assert launches((0,), 8960, 2048, 1) < 0          # bad shape: an error code
