"""Reading (and writing) NF4 weights in the layout transformers + bitsandbytes store in a 4-bit
checkpoint, so that the kernels can run on weights quantised elsewhere.

The reference never parses that layout itself: it gets live `QuantState` objects from
bitsandbytes after `from_pretrained` (harness/eval_adapter.py:26-35; solution/packed.py:57-79 reads
their fields). bitsandbytes is not installed here and the reference holds no serialized sample, so
the key names below follow bitsandbytes' published `QuantState.as_dict(packed=True)` /
`QuantState.from_dict` and are NOT pinned against a real checkpoint: parity unpinned.

Per `Linear4bit` weight `<prefix>` (for example `model.layers.0.mlp.gate_proj.weight`):
    <prefix>                                    uint8 [n*k/2, 1]   two codes per byte
    <prefix>.absmax                             uint8 [n*k/64] (double quant) or fp32 [n*k/64]
    <prefix>.quant_map                          fp32 [16]          the NF4 table
    <prefix>.nested_absmax                      fp32 [n*k/64/256]  (double quant only)
    <prefix>.nested_quant_map                   fp32 [256]         (double quant only)
    <prefix>.quant_state.bitsandbytes__nf4      uint8 [*]          UTF-8 JSON: quant_type, blocksize,
                                                                   dtype, shape, nested_blocksize,
                                                                   nested_dtype, nested_offset
"""

from __future__ import annotations

import json
from typing import Dict, Mapping, Tuple

import torch

from .quantize import NestedState, QuantState

_DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
_META_KEY = ".quant_state.bitsandbytes__nf4"


def is_nf4_weight(tensors: Mapping[str, torch.Tensor], prefix: str) -> bool:
    return prefix in tensors and prefix + _META_KEY in tensors


def quant_state_from_dict(tensors: Mapping[str, torch.Tensor], prefix: str,
                          device="cpu") -> Tuple[torch.Tensor, QuantState]:
    """(packed codes, QuantState) of the weight stored under `prefix`."""
    if not is_nf4_weight(tensors, prefix):
        raise KeyError(f"hackaton_b200: no NF4 weight under {prefix!r}")
    meta = json.loads(bytes(tensors[prefix + _META_KEY].cpu().numpy().tobytes()).decode("utf-8"))
    if meta.get("quant_type") != "nf4":
        raise ValueError(f"hackaton_b200: {prefix}: quant_type {meta.get('quant_type')!r}, only nf4 is handled")
    shape = tuple(int(v) for v in meta["shape"])
    dtype = _DTYPES[str(meta["dtype"]).replace("torch.", "")]
    packed = tensors[prefix].to(device).reshape(-1).contiguous()
    if packed.dtype != torch.uint8 or packed.numel() * 2 != shape[0] * shape[1]:
        raise ValueError(f"hackaton_b200: {prefix}: {packed.numel()} code bytes for shape {shape}")
    absmax = tensors[prefix + ".absmax"].to(device).contiguous()
    code = tensors[prefix + ".quant_map"].to(device=device, dtype=torch.float32).contiguous()
    nested = prefix + ".nested_absmax" in tensors
    state2 = offset = None
    if nested:
        state2 = NestedState(
            absmax=tensors[prefix + ".nested_absmax"].to(device=device, dtype=torch.float32).contiguous(),
            code=tensors[prefix + ".nested_quant_map"].to(device=device, dtype=torch.float32).contiguous(),
            blocksize=int(meta["nested_blocksize"]))
        offset = torch.tensor(float(meta["nested_offset"]), dtype=torch.float32, device=device)
        if absmax.dtype != torch.uint8:
            raise ValueError(f"hackaton_b200: {prefix}: nested state with {absmax.dtype} absmax")
    elif absmax.dtype != torch.float32:
        absmax = absmax.float()
    state = QuantState(absmax=absmax, code=code, shape=shape, dtype=dtype, blocksize=int(meta["blocksize"]),
                       quant_type="nf4", nested=nested, state2=state2, offset=offset)
    return packed, state


def quant_state_to_dict(packed: torch.Tensor, state: QuantState, prefix: str) -> Dict[str, torch.Tensor]:
    """The inverse: the tensors a checkpoint would hold for this weight."""
    meta = {"quant_type": "nf4", "blocksize": int(state.blocksize),
            "dtype": str(state.dtype).replace("torch.", ""), "shape": [int(v) for v in state.shape]}
    out = {prefix: packed.detach().cpu().reshape(-1, 1).contiguous(),
           prefix + ".absmax": state.absmax.detach().cpu().contiguous(),
           prefix + ".quant_map": state.code.detach().cpu().float().contiguous()}
    if state.nested:
        out[prefix + ".nested_absmax"] = state.state2.absmax.detach().cpu().contiguous()
        out[prefix + ".nested_quant_map"] = state.state2.code.detach().cpu().contiguous()
        meta.update({"nested_blocksize": int(state.state2.blocksize), "nested_dtype": "float32",
                     "nested_offset": float(state.offset)})
    raw = json.dumps(meta).encode("utf-8")
    out[prefix + _META_KEY] = torch.frombuffer(bytearray(raw), dtype=torch.uint8).clone()
    return out


def load_nf4_weights(path: str, device="cpu") -> Dict[str, Tuple[torch.Tensor, QuantState]]:
    """All NF4 weights of a `.safetensors` file: {weight name: (packed, QuantState)}."""
    from safetensors import safe_open

    found = {}
    with safe_open(path, framework="pt", device="cpu") as f:
        keys = set(f.keys())
        for key in sorted(keys):
            if not key.endswith(_META_KEY):
                continue
            prefix = key[: -len(_META_KEY)]
            names = [prefix, key, prefix + ".absmax", prefix + ".quant_map"]
            names += [n for n in (prefix + ".nested_absmax", prefix + ".nested_quant_map") if n in keys]
            found[prefix] = quant_state_from_dict({n: f.get_tensor(n) for n in names}, prefix, device)
    return found
