"""Patches that route bitsandbytes' 4-bit matmul and peft's LoRA-on-4-bit forward through the
B200 kernels: the plug-in boundary of the reference (solution/patches.py:251-277 and
solution/__init__.py:23-33), for the NF4 path only.

As in the reference, a call the kernels do not cover goes to the function that was there before
the patch (bitsandbytes' or peft's own code), never to a CPU path of this package.
"""

from __future__ import annotations

import torch

from .lora import RANK, nf4_lora_linear
from .nf4 import can_dequantize, nf4_linear


def _is_4bit_linear(module):
    """solution/patches.py:12-17."""
    try:
        import bitsandbytes as bnb
    except ImportError:
        return False
    return isinstance(module, bnb.nn.Linear4bit)


def _eligible(A, state, packed, bias):
    """The reference's guard (solution/patches.py:266-272) without its two T4-only limits: the
    minimum weight size (MIN_NF4_WEIGHTS, there to save per-launch CPU time in the contest) and
    the "more than 4 rows" rule (small batches take the same fused kernel here). Nested states
    are accepted; the compute dtype must be fp16 and K a multiple of 64."""
    return (state is not None and isinstance(A, torch.Tensor) and A.is_cuda and A.dim() >= 2
            and len(getattr(state, "shape", ())) == 2 and A.shape[-1] == state.shape[1]
            and A.dtype == torch.float16 and getattr(state, "dtype", None) == torch.float16
            and getattr(state, "blocksize", 0) == 64 and state.shape[1] % 64 == 0
            and can_dequantize(packed.reshape(-1), state)
            and (bias is None or bias.dtype == A.dtype))


def _plain_lora_adapter(module, name, state):
    """True when adapter `name` of a peft LoRA wrapper is the plain update the fused kernel
    computes, base(x) + scaling * B(A(dropout(x))): rank 16, no bias on either factor, A reading
    the base layer's input features, and none of peft's variants that change the formula
    (DoRA's magnitude vector, entries of `lora_variant`). Anything else must take peft's own
    forward: computing plain LoRA for such an adapter would be silently wrong."""
    if name not in getattr(module, "lora_A", {}) or name not in getattr(module, "lora_B", {}):
        return False
    use_dora = getattr(module, "use_dora", None)
    if isinstance(use_dora, dict) and use_dora.get(name):
        return False
    for attr in ("lora_variant", "lora_magnitude_vector"):
        table = getattr(module, attr, None)
        if table is not None and name in table:
            return False
    a_mod, b_mod = module.lora_A[name], module.lora_B[name]
    lora_a, lora_b = getattr(a_mod, "weight", None), getattr(b_mod, "weight", None)
    if lora_a is None or lora_b is None or lora_a.dim() != 2 or lora_b.dim() != 2:
        return False
    return (lora_a.shape[0] == RANK and lora_b.shape[1] == RANK
            and lora_a.shape[1] == state.shape[1] and lora_b.shape[0] == state.shape[0]
            and getattr(a_mod, "bias", None) is None and getattr(b_mod, "bias", None) is None)


def patch_nf4_matmul():
    """Replaces `bitsandbytes.matmul_4bit(A, B, quant_state, out=None, bias=None)` (the call every
    `Linear4bit.forward` makes) by the fused NF4 linear; see solution/patches.py:251-277."""
    import bitsandbytes as bnb

    original = bnb.matmul_4bit
    if getattr(original, "_nf4b200", False):
        return

    def matmul_4bit(A, B, quant_state, out=None, bias=None):
        if out is None and _eligible(A, quant_state, B, bias):
            return nf4_linear(A, B, bias, quant_state)
        return original(A, B, quant_state, out=out, bias=bias)

    matmul_4bit._nf4b200 = True
    matmul_4bit._original = original
    bnb.matmul_4bit = matmul_4bit


def lora_forward_for(original):
    """Builds the replacement for peft's `lora.bnb.Linear4bit.forward`. Module attributes used:
    `base_layer` (a bnb `Linear4bit`: `.weight` with `.quant_state`, `.bias`), `lora_A`,
    `lora_B`, `lora_dropout`, `scaling` (dicts keyed by adapter name), `active_adapters`,
    `disable_adapters`, `merged` (names as in the reference's tools/probe.py:127-129)."""

    def forward(self, x, *args, **kwargs):
        adapters = list(getattr(self, "active_adapters", ()))
        base = getattr(self, "base_layer", None)
        weight = getattr(base, "weight", None)
        state = getattr(weight, "quant_state", None)
        if (args or kwargs or getattr(self, "disable_adapters", False)
                or getattr(self, "merged", False) or len(adapters) != 1
                or adapters[0] not in self.lora_A or weight is None
                or not _eligible(x, state, weight, getattr(base, "bias", None))):
            return original(self, x, *args, **kwargs)
        name = adapters[0]
        if not _plain_lora_adapter(self, name, state):
            return original(self, x, *args, **kwargs)
        lora_a, lora_b = self.lora_A[name].weight, self.lora_B[name].weight
        dropout = self.lora_dropout[name]
        x_lora = dropout(x) if (dropout.training and getattr(dropout, "p", 0.0) > 0.0) else x
        return nf4_lora_linear(x, weight, base.bias, state, lora_a, lora_b,
                               float(self.scaling[name]), x_lora=x_lora)

    forward._nf4b200 = True
    forward._original = original
    return forward


def patch_peft_lora():
    """Replaces the forward of peft's LoRA wrapper around 4-bit linears by the fused kernel."""
    try:
        from peft.tuners.lora import bnb as peft_bnb
    except ImportError:
        return
    cls = getattr(peft_bnb, "Linear4bit", None)
    if cls is None or getattr(cls.forward, "_nf4b200", False):
        return
    cls.forward = lora_forward_for(cls.forward)


class SiblingGroup:
    """Projections that are fed the same tensor (q/k/v of an attention block, gate/up of an MLP:
    the call sites solution/patches.py:32-41 and :98-99 of the reference), run as one grouped
    launch without touching the code that calls them.

    After `install()`, the first of the modules to be called with a tensor x computes the outputs
    of all of them (`nf4_linear_group`: one fused kernel forward, one summed dX backward) and
    keeps the siblings' shares; when a sibling is then called with the very same x it returns its
    share. Anything the grouped kernel does not cover (a call with extra arguments, an input that
    is not eligible, an adapter with active dropout, merged or disabled adapters, a rank other
    than 16) goes to the module's own forward, as everywhere in this file.

    Members may be bitsandbytes `Linear4bit` modules or peft LoRA wrappers around them
    (attributes as in `lora_forward_for`)."""

    def __init__(self, modules):
        self.modules = list(modules)
        self.originals = [m.forward for m in self.modules]
        self._x = None
        self._shares = {}

    def install(self):
        for i, m in enumerate(self.modules):
            m.forward = self._forward_for(i)
        return self

    def remove(self):
        for m, f in zip(self.modules, self.originals):
            m.forward = f
        self._x, self._shares = None, {}

    def _forward_for(self, index):
        def forward(x, *args, **kwargs):
            return self._call(index, x, *args, **kwargs)
        forward._nf4b200 = True
        return forward

    def _projection(self, module, x):
        from .group import Projection

        base = getattr(module, "base_layer", module)
        weight = getattr(base, "weight", None)
        state = getattr(weight, "quant_state", None)
        bias = getattr(base, "bias", None)
        if weight is None or not _eligible(x, state, weight, bias):
            return None
        if not hasattr(module, "lora_A"):
            return Projection(weight, state, bias)
        adapters = list(getattr(module, "active_adapters", ()))
        if (getattr(module, "disable_adapters", False) or getattr(module, "merged", False)
                or len(adapters) != 1 or adapters[0] not in module.lora_A):
            return None
        name = adapters[0]
        if not _plain_lora_adapter(module, name, state):
            return None
        lora_a, lora_b = module.lora_A[name].weight, module.lora_B[name].weight
        dropout = module.lora_dropout[name]
        if getattr(dropout, "training", False) and getattr(dropout, "p", 0.0) > 0.0:
            return None
        return Projection(weight, state, bias, lora_a, lora_b, float(module.scaling[name]))

    def _call(self, index, x, *args, **kwargs):
        if args or kwargs:
            return self.originals[index](x, *args, **kwargs)
        if self._x is x and index in self._shares:
            y = self._shares.pop(index)
            if not self._shares:
                self._x = None
            return y
        projections = [self._projection(m, x) for m in self.modules]
        if any(p is None for p in projections):
            return self.originals[index](x)
        from . import group as _group
        ys = _group.nf4_linear_group(x, projections)
        self._x = x
        self._shares = {i: y for i, y in enumerate(ys) if i != index}
        return ys[index]


SIBLINGS = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))


def patch_sibling_projections(model):
    """Walks `model.modules()` and groups, inside every block that has them, q_proj/k_proj/v_proj
    and gate_proj/up_proj (the attribute names of transformers' Qwen2 attention and MLP blocks)
    when all members are 4-bit linears or LoRA wrappers around 4-bit linears with the same number
    of input features. Returns the installed groups (call `.remove()` on them to undo)."""
    groups = []
    for block in model.modules():
        for names in SIBLINGS:
            members = [getattr(block, n, None) for n in names]
            if any(m is None for m in members):
                continue
            bases = [getattr(m, "base_layer", m) for m in members]
            if not all(_is_4bit_linear(b) for b in bases):
                continue
            if len({getattr(b, "in_features", None) for b in bases}) != 1:
                continue
            if any(getattr(m.forward, "_nf4b200", False) for m in members):
                continue   # already grouped
            groups.append(SiblingGroup(members).install())
    return groups


def mlp_forward_for(original):
    """Builds the replacement for `Qwen2MLP.forward` (the reference's `patch_qwen2_mlp`,
    solution/patches.py:20-43): the input is cast to fp16 once, gate_proj, up_proj and the SwiGLU
    product run as one fused kernel and down_proj takes the fp16 product (`nf4_swiglu_mlp`, whose
    backward also folds the SwiGLU backward into down_proj's dX kernel; `nf4_gate_up_swiglu` +
    the module's own forward when down_proj is not eligible), and the result goes back to the
    stream's dtype. Same conditions as the reference (silu
    activation, CUDA input, three plain 4-bit linears) plus this library's own (`_eligible`);
    everything else runs the original forward."""
    from .group import Projection
    from . import mlp as _mlp

    def forward(self, x):
        gate_proj, up_proj, down_proj = self.gate_proj, self.up_proj, self.down_proj
        act = getattr(getattr(self, "config", None), "hidden_act", "silu")
        if (act != "silu" or not isinstance(x, torch.Tensor) or not x.is_cuda
                or not all(_is_4bit_linear(m) for m in (gate_proj, up_proj, down_proj))):
            return original(self, x)
        compute = getattr(gate_proj, "compute_dtype", None) or torch.float16
        if compute != torch.float16:
            return original(self, x)
        x16 = x.to(compute)
        states = [getattr(m.weight, "quant_state", None) for m in (gate_proj, up_proj)]
        if not all(_eligible(x16, st, m.weight, None) and getattr(m, "bias", None) is None
                   for m, st in zip((gate_proj, up_proj), states)) \
                or tuple(states[0].shape) != tuple(states[1].shape):
            return original(self, x)
        gate_p, up_p = Projection(gate_proj.weight, states[0]), Projection(up_proj.weight, states[1])
        down_state = getattr(down_proj.weight, "quant_state", None)
        if (getattr(down_proj, "bias", None) is None and down_state is not None
                and len(getattr(down_state, "shape", ())) == 2
                and down_state.shape[1] == states[0].shape[0]
                and _eligible(x16.new_empty((1, down_state.shape[1])), down_state,
                              down_proj.weight, None)):
            return _mlp.nf4_swiglu_mlp(x16, gate_p, up_p,
                                       Projection(down_proj.weight, down_state)).to(x.dtype)
        hidden = _mlp.nf4_gate_up_swiglu(x16, gate_p, up_p)
        return down_proj(hidden).to(x.dtype)

    forward._nf4b200 = True
    forward._original = original
    return forward


def patch_qwen2_mlp():
    """Installs `mlp_forward_for` on transformers' Qwen2MLP. Not part of `apply()`: the reference
    installs its MLP patch from `solution.apply()` together with a dozen others; here it is an
    explicit opt-in next to the two patches of the GEMM path."""
    try:
        from transformers.models.qwen2 import modeling_qwen2
    except ImportError:
        return False
    current = modeling_qwen2.Qwen2MLP.forward
    if getattr(current, "_nf4b200", False):
        return True
    modeling_qwen2.Qwen2MLP.forward = mlp_forward_for(current)
    return True


def apply():
    """The entry point the reference's harness calls once before the model is built
    (solution/__init__.py:23-33), restricted to the NF4 path."""
    patch_nf4_matmul()
    patch_peft_lora()
