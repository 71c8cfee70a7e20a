"""hackaton_b200: the NF4 (bitsandbytes layout, double quant) dequant-GEMM-LoRA hot path of
mergentlegen/hackaton as hand-written sm_100a CUDA kernels behind the reference's Python surface.

    from hackaton_b200 import dequantize_nf4, nf4_linear, nf4_lora_linear, apply
"""

from .group import Projection, nf4_linear_group
from .lora import NF4LoRALinear, nf4_lora_linear
from .mlp import nf4_gate_up_swiglu, silu_mul
from .nf4 import NF4Linear, can_dequantize, dequantize_nf4, nf4_linear
from .patches import apply, patch_nf4_matmul, patch_peft_lora
from .quantize import QuantState, quantize_nf4

__all__ = [
    "NF4Linear", "NF4LoRALinear", "Projection", "QuantState", "apply", "can_dequantize",
    "dequantize_nf4", "nf4_gate_up_swiglu", "nf4_linear", "nf4_linear_group", "nf4_lora_linear", "patch_nf4_matmul",
    "patch_peft_lora", "quantize_nf4", "silu_mul",
]
