"""hackaton_b200: the NF4 (bitsandbytes layout, double quant) dequant-GEMM-LoRA hot path of
mergentlegen/hackaton as hand-written sm_100a CUDA kernels behind the reference's Python surface.

    from hackaton_b200 import dequantize_nf4, nf4_linear, nf4_lora_linear, apply
"""

from .dense import fp16_linear
from .group import Projection, nf4_linear_group
from .lora import NF4LoRALinear, nf4_lora_linear
from .lm_loss import fused_cross_entropy, linear_cross_entropy
from .mlp import nf4_gate_up_swiglu, nf4_swiglu_mlp, silu_mul
from .nf4 import NF4Linear, can_dequantize, dequantize_nf4, nf4_linear
from .patches import apply, patch_nf4_matmul, patch_peft_lora
from .quantize import QuantState, quantize_nf4
from .rmsnorm import add_rms_norm, rms_norm
from .rope import qkv_rotate

__all__ = [
    "NF4Linear", "NF4LoRALinear", "Projection", "QuantState", "add_rms_norm", "apply", "can_dequantize",
    "dequantize_nf4", "fp16_linear", "fused_cross_entropy", "linear_cross_entropy", "nf4_gate_up_swiglu", "nf4_linear",
    "nf4_linear_group", "nf4_lora_linear", "nf4_swiglu_mlp", "patch_nf4_matmul",
    "patch_peft_lora", "qkv_rotate", "quantize_nf4", "rms_norm", "silu_mul",
]
