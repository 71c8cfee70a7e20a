"""CPU: the bitsandbytes-layout checkpoint reader: a weight written in that layout to a
.safetensors file comes back with the same codes, tables and scalars, and decodes to the same
values. (Key names follow bitsandbytes' published QuantState.as_dict; no real checkpoint is
available here to pin them against.)"""

import json

import pytest
import torch

from oracle import nf4_oracle
from tests.util import oracle_weight, synthetic_weight


@pytest.mark.parametrize("nested", [True, False])
def test_round_trip_through_safetensors(tmp_path, nested):
    from safetensors.torch import save_file

    from hackaton_b200.checkpoint import is_nf4_weight, load_nf4_weights, quant_state_to_dict

    tensors = {"model.norm.weight": torch.ones(8)}
    originals = {}
    for i, (rows, cols) in enumerate([(96, 192), (24, 128)]):
        packed, state = synthetic_weight(rows, cols, nested, seed=3 + i)
        name = f"model.layers.{i}.mlp.gate_proj.weight"
        originals[name] = (packed, state)
        tensors.update(quant_state_to_dict(packed, state, name))
    assert is_nf4_weight(tensors, "model.layers.0.mlp.gate_proj.weight")
    assert not is_nf4_weight(tensors, "model.norm.weight")
    meta = json.loads(bytes(tensors["model.layers.0.mlp.gate_proj.weight.quant_state.bitsandbytes__nf4"]
                            .numpy().tobytes()).decode())
    assert meta["quant_type"] == "nf4" and meta["blocksize"] == 64 and meta["shape"] == [96, 192]
    assert ("nested_offset" in meta) == nested
    path = tmp_path / "model.safetensors"
    save_file(tensors, str(path))
    loaded = load_nf4_weights(str(path))
    assert sorted(loaded) == sorted(originals)
    for name, (packed, state) in originals.items():
        got_packed, got = loaded[name]
        assert torch.equal(got_packed, packed.reshape(-1))
        assert got.shape == tuple(state.shape) and got.dtype == state.dtype and got.nested == nested
        assert got.blocksize == state.blocksize and torch.equal(got.absmax, state.absmax)
        assert torch.equal(got.code, state.code)
        if nested:
            assert torch.equal(got.state2.absmax, state.state2.absmax)
            assert torch.equal(got.state2.code, state.state2.code)
            assert got.state2.blocksize == state.state2.blocksize
            assert float(got.offset) == float(state.offset)
        assert torch.equal(oracle_weight(got_packed, got).view(torch.int16),
                           oracle_weight(packed, state).view(torch.int16))


def test_rejects_other_formats():
    from hackaton_b200.checkpoint import quant_state_from_dict, quant_state_to_dict

    packed, state = synthetic_weight(16, 64, True, seed=1)
    tensors = quant_state_to_dict(packed, state, "w")
    with pytest.raises(KeyError):
        quant_state_from_dict(tensors, "missing")
    bad = dict(tensors)
    raw = json.dumps({"quant_type": "fp4", "blocksize": 64, "dtype": "float16", "shape": [16, 64]}).encode()
    bad["w.quant_state.bitsandbytes__nf4"] = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
    with pytest.raises(ValueError):
        quant_state_from_dict(bad, "w")
    short = dict(tensors)
    short["w"] = tensors["w"][:-1]
    with pytest.raises(ValueError):
        quant_state_from_dict(short, "w")
