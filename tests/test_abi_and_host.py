"""CPU: the C-ABI library builds, loads and exports every symbol include/nf4b200.h declares;
host-side guards and patches behave like the reference's (no compute calls here)."""

import ctypes
import re
import sys
import types
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def library():
    from hackaton_b200.build import build_library

    return ctypes.CDLL(str(build_library()))


def declared_functions():
    text = (ROOT / "include" / "nf4b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nf4b200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(library):
    names = declared_functions()
    assert len(names) >= 8
    for name in names:
        assert hasattr(library, name), f"{name} declared in nf4b200.h but not exported"


def test_binding_covers_the_header():
    from hackaton_b200 import _lib

    assert sorted(_lib.EXPORTS) == declared_functions()


def test_struct_layout_matches_header():
    from hackaton_b200 import _lib

    assert ctypes.sizeof(_lib.Weight) == 6 * 8 + 2 * 8 + 4 * 4 + 8
    assert _lib.Weight.scales16.offset == 80
    assert ctypes.sizeof(_lib.Props) == 4 * 4 + 8


def test_no_gpu_means_error_not_fallback(library):
    """Without a CUDA device every compute entry point reports an error status."""
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from hackaton_b200 import _lib

    w = _lib.Weight()
    rc = _lib.lib().nf4b200_dequant(ctypes.byref(w), None, 0, None)
    assert rc != 0
    assert _lib.lib().nf4b200_last_error()


def test_can_dequantize_guards():
    from hackaton_b200 import can_dequantize
    from tests.util import synthetic_weight

    packed, state = synthetic_weight(8, 64, True)
    assert not can_dequantize(packed, state)           # CPU tensors: never eligible
    assert not can_dequantize("not a tensor", state)


def test_product_does_not_import_the_oracle():
    for path in (ROOT / "hackaton_b200").rglob("*.py"):
        text = path.read_text()
        assert "oracle" not in re.sub(r'""".*?"""', "", text, flags=re.S), path


def test_matmul_patch_falls_through_to_original(monkeypatch):
    """solution/patches.py:266-275: whatever the kernels do not cover goes to the function that
    was installed before (here a fake bitsandbytes)."""
    calls = []
    fake = types.ModuleType("bitsandbytes")
    fake.matmul_4bit = lambda A, B, quant_state, out=None, bias=None: calls.append("orig") or "orig"
    fake.nn = types.SimpleNamespace(Linear4bit=type("Linear4bit", (), {}))
    monkeypatch.setitem(sys.modules, "bitsandbytes", fake)
    from hackaton_b200 import patches

    patches.patch_nf4_matmul()
    patched = fake.matmul_4bit
    assert patched._nf4b200
    patches.patch_nf4_matmul()                      # idempotent
    assert fake.matmul_4bit is patched
    x = torch.zeros(8, 64, dtype=torch.float16)     # CPU tensor -> not eligible
    assert fake.matmul_4bit(x, torch.zeros(1, 8, dtype=torch.uint8), None) == "orig"
    assert calls == ["orig"]
    assert patches._is_4bit_linear(fake.nn.Linear4bit())
    assert not patches._is_4bit_linear(object())


def test_lora_patch_falls_through_to_original():
    from hackaton_b200 import patches

    seen = []
    forward = patches.lora_forward_for(lambda self, x, *a, **k: seen.append(1) or "orig")
    module = types.SimpleNamespace(active_adapters=["default"], disable_adapters=True,
                                   merged=False, base_layer=None, lora_A={}, lora_B={})
    assert forward(module, torch.zeros(2, 64)) == "orig" and seen == [1]


def _fake_lora_module(k=128, n=64, rank=16, **extra):
    """A stand-in for peft's LoRA wrapper around a 4-bit linear, with the attributes the patch reads."""
    state = types.SimpleNamespace(shape=(n, k))
    base = types.SimpleNamespace(weight=types.SimpleNamespace(quant_state=state), bias=None)
    mod = types.SimpleNamespace(
        active_adapters=["default"], disable_adapters=False, merged=False, base_layer=base,
        lora_A={"default": types.SimpleNamespace(weight=torch.zeros(rank, k), bias=None)},
        lora_B={"default": types.SimpleNamespace(weight=torch.zeros(n, rank), bias=None)},
        lora_dropout={"default": torch.nn.Identity()}, scaling={"default": 2.0},
        forward=lambda x: "own")
    for key, value in extra.items():
        setattr(mod, key, value)
    return mod


@pytest.mark.parametrize("extra,fused", [
    ({}, True),
    ({"use_dora": {"default": True}}, False),                 # DoRA: another formula
    ({"use_dora": {"default": False}}, True),
    ({"lora_variant": {"default": object()}}, False),          # newer peft: any registered variant
    ({"lora_magnitude_vector": {"default": object()}}, False),
    ({"lora_variant": {}, "lora_magnitude_vector": {}}, True),
])
def test_lora_patch_leaves_adapter_variants_to_peft(monkeypatch, extra, fused):
    """Adapters whose forward is not the plain low-rank update (DoRA, entries of `lora_variant`)
    take peft's own forward, in the module patch and in the sibling groups alike."""
    from hackaton_b200 import patches

    monkeypatch.setattr(patches, "_eligible", lambda x, state, weight, bias: True)
    monkeypatch.setattr(patches, "nf4_lora_linear", lambda *a, **k: "fused")
    forward = patches.lora_forward_for(lambda self, x, *a, **k: "orig")
    module = _fake_lora_module(**extra)
    assert forward(module, torch.zeros(2, 128)) == ("fused" if fused else "orig")
    proj = patches.SiblingGroup([module])._projection(module, torch.zeros(2, 128))
    assert (proj is not None) == fused


def test_lora_patch_checks_rank_and_feature_counts(monkeypatch):
    from hackaton_b200 import patches

    monkeypatch.setattr(patches, "_eligible", lambda x, state, weight, bias: True)
    monkeypatch.setattr(patches, "nf4_lora_linear", lambda *a, **k: "fused")
    forward = patches.lora_forward_for(lambda self, x, *a, **k: "orig")
    assert forward(_fake_lora_module(rank=8), torch.zeros(2, 128)) == "orig"
    wrong_in = _fake_lora_module()
    wrong_in.lora_A["default"].weight = torch.zeros(16, 64)     # A does not read the base input
    assert forward(wrong_in, torch.zeros(2, 128)) == "orig"
    biased = _fake_lora_module()
    biased.lora_B["default"].bias = torch.zeros(64)
    assert forward(biased, torch.zeros(2, 128)) == "orig"


def test_sibling_group_routes_one_launch(monkeypatch):
    """q/k/v called one after the other with the same tensor: one grouped computation, every
    module gets its own share; another tensor, or an ineligible input, starts over or falls
    through to the module's own forward."""
    import types

    from hackaton_b200 import group, patches

    class Lin(torch.nn.Module):
        def __init__(self, tag):
            super().__init__()
            self.tag = tag
            self.weight = types.SimpleNamespace(quant_state=object())
            self.bias = None

        def forward(self, x):
            return ("own", self.tag)

    calls = []

    def fake_group(x, projections):
        calls.append(len(projections))
        return [("grouped", i, id(x)) for i in range(len(projections))]

    eligible = {"ok": True}
    monkeypatch.setattr(patches, "_eligible", lambda x, state, weight, bias: eligible["ok"])
    monkeypatch.setattr(group, "nf4_linear_group", fake_group)
    q, k, v = Lin("q"), Lin("k"), Lin("v")
    g = patches.SiblingGroup([q, k, v]).install()
    x = torch.zeros(2, 4)
    assert q(x) == ("grouped", 0, id(x))
    assert v(x) == ("grouped", 2, id(x))
    assert k(x) == ("grouped", 1, id(x))
    assert calls == [3]
    x2 = torch.zeros(2, 4)
    assert k(x2) == ("grouped", 1, id(x2)) and calls == [3, 3]
    assert k(x2) == ("grouped", 1, id(x2)) and calls == [3, 3, 3]   # its share was already taken
    eligible["ok"] = False
    assert q(torch.zeros(2, 4)) == ("own", "q")
    g.remove()
    eligible["ok"] = True
    assert q(x) == ("own", "q")


def test_patch_sibling_projections_finds_blocks(monkeypatch):
    import types

    from hackaton_b200 import patches

    class Lin(torch.nn.Module):
        def __init__(self, n_in):
            super().__init__()
            self.in_features = n_in

        def forward(self, x):
            return x

    monkeypatch.setattr(patches, "_is_4bit_linear", lambda m: isinstance(m, Lin))

    class Attn(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj, self.k_proj, self.v_proj, self.o_proj = Lin(8), Lin(8), Lin(8), Lin(8)

    class Mlp(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj, self.up_proj, self.down_proj = Lin(8), Lin(8), Lin(16)

    model = torch.nn.Sequential(Attn(), Mlp(), Attn())
    groups = patches.patch_sibling_projections(model)
    assert [len(g.modules) for g in groups] == [3, 2, 3]
    assert patches.patch_sibling_projections(model) == []      # nothing left to group
    for g in groups:
        g.remove()


def test_mlp_patch_routes_and_falls_through(monkeypatch):
    """The Qwen2MLP replacement: eligible 4-bit gate/up go through the fused front half and
    down_proj sees its fp16 result; another activation, or an ineligible input, runs the
    original forward (solution/patches.py:32-41 has the same shape)."""
    import types

    from hackaton_b200 import mlp, patches

    class Lin(torch.nn.Module):
        def __init__(self, tag):
            super().__init__()
            self.tag = tag
            self.weight = types.SimpleNamespace(quant_state=types.SimpleNamespace(shape=(8, 4)))
            self.bias = None
            self.compute_dtype = torch.float16

        def forward(self, x):
            return ("down", x)

    class Mlp:
        def __init__(self, act="silu"):
            self.gate_proj, self.up_proj, self.down_proj = Lin("g"), Lin("u"), Lin("d")
            self.config = types.SimpleNamespace(hidden_act=act)

    class FakeCuda(torch.Tensor):
        is_cuda = True

    calls = []

    def fake_front(x16, gate, up):
        calls.append((x16.dtype, gate.packed, up.packed))
        return torch.ones(2, 8, dtype=torch.float16)

    class Out:
        def __init__(self, v):
            self.v = v

        def to(self, dtype):
            return ("cast", dtype, self.v)

    monkeypatch.setattr(patches, "_is_4bit_linear", lambda m: isinstance(m, Lin))
    monkeypatch.setattr(patches, "_eligible", lambda x, state, weight, bias: True)
    monkeypatch.setattr(mlp, "nf4_gate_up_swiglu", fake_front)
    monkeypatch.setattr(Lin, "forward", lambda self, x: Out(("down", tuple(x.shape), x.dtype)))
    forward = patches.mlp_forward_for(lambda self, x: "original")
    x = torch.zeros(2, 4, dtype=torch.float32).as_subclass(FakeCuda)
    block = Mlp()
    assert forward(block, x) == ("cast", torch.float32, ("down", (2, 8), torch.float16))
    assert calls == [(torch.float16, block.gate_proj.weight, block.up_proj.weight)]
    assert forward(Mlp("gelu"), x) == "original"
    assert forward(block, torch.zeros(2, 4)) == "original"            # not on a GPU
    monkeypatch.setattr(patches, "_eligible", lambda x, state, weight, bias: False)
    assert forward(block, x) == "original"
    assert len(calls) == 1
