"""CPU oracle for the hot path: TEST INFRASTRUCTURE, never the product.

Everything here is a CPU restatement (NumPy, and C in cpu_ref.c) of the math
the reference runs for this path: the quantisers and quantised products of
examples/llm/qwen3.py, its RMSNorm / softmax / RoPE / decode attention /
decoder forward, the bench-form LayerNorm of bench/jax_bench.py, and the GEMM
epilogue formulas of metal_pjrt/kernels/steel_gemm.metal.  Only the tests,
the smoke check and the benchmark's CPU-baseline leg may import it; the
library never does, and has no CPU fallback.

Pinning.  The reference holds no golden vectors for this path (every one of
its comparisons is against a freshly computed CPU result with a tolerance).
What pins this oracle:
  * tests/golden/*.npz, produced by tests/golden/make_golden.py, which imports
    the reference's own examples/llm/qwen3.py (with NumPy standing in for the
    absent jax module) and records its quantisers, quantised products,
    rms_norm, rope, decode attention and a small decoder forward;
  * the bf16 rounding rule and activation formulas written out in the
    reference's own unit tests (blas/steel_gemm_test.cc:30-41,
    blas/gemv_test.cc:66-74).
The BASELINE variants of the quantisers (per-channel int8; min/max affine
int4 packed eight nibbles per uint32) have no reference code at all: for
them parity is UNPINNED beyond self-consistency (pack -> unpack -> dequant
round trips and agreement between the NumPy and the C restatement).
XLA:CPU's own summation order is likewise unpinned (jaxlib is absent here).
"""
from . import dense, quant, rownorm, decoder, inputs  # noqa: F401
