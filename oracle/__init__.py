"""CPU oracle for the NF4 dequant + linear + LoRA path.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this; only the tests, the smoke
check and the CPU-baseline leg of the benchmark do, and there only as the checker / the timed CPU
baseline, never as a fallback for the CUDA kernels.

Parity status
-------------
* flat-scale decode: pinned against the reference's own `nf4_dequant_kernel`
  (solution/nf4.py:28-44) run on CPU under the Triton interpreter; golden vectors and digests are
  committed under tests/golden/ together with the script that made them.
* linear forward / backward: pinned against the reference's `NF4Linear` (solution/nf4.py:80-102)
  run on CPU tensors through the same interpreter path (golden vectors, fp16 tolerance).
* nested (double-quantised) absmax and LoRA: parity unpinned. The reference delegates the nested
  decode to bitsandbytes==0.50.2 (`dequantize_blockwise`, solution/packed.py:74-77) and LoRA to
  peft==0.20.0; neither is vendored nor installed. The oracle restates their published
  arithmetic: `code2[u8] * absmax2[i // 256]`, then `+ offset`, two separately rounded fp32 ops;
  `y = base(x) + (x Aᵀ Bᵀ) * (alpha / r)`.
* SwiGLU (solution/kernels.py:39-57), RMSNorm in its four modes (solution/rmsnorm.py:17-49), the
  q/k/v rotation with grouped-query expansion (solution/attention.py:36-146) and the
  cross-entropy statistics / gradient (solution/kernels.py:106-165): pinned against the
  reference's own kernels run on CPU under the Triton interpreter (tests/golden/make_golden_*.py,
  vectors committed beside the scripts).
"""
