"""Oracle: dense GEMM with the fused epilogue (test infrastructure).

Restates, on the CPU in float64, what the reference's GEMM kernels compute
per output element (metal_pjrt/kernels/steel_gemm.metal:58-66,217-225 and the
unit-test reference loops blas/steel_gemm_test.cc:160-196,
blas/gemv_test.cc:66-74):

    v   = alpha * sum_k op(A)[i,k] * op(B)[k,j]  (+ beta * C[i,j])  (+ bias[j])
    aux = round(v)            when an aux output is asked for
    D   = round(act(v))       act in {none, ReLU (keeps NaN), GELU-tanh, SiLU}

with one rounding to the output dtype.
"""
import ml_dtypes
import numpy as np

bf16 = ml_dtypes.bfloat16

ACT_NONE, ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2, 3
_GELU_K = 0.7978845608028654  # sqrt(2/pi), steel_gemm.metal:61


def act(kind, v):
    """Activation in float64 (blas/gemv_test.cc:66-74); ReLU keeps NaN
    (steel_gemm.metal:59)."""
    v = np.asarray(v, np.float64)
    if kind == ACT_RELU:
        return np.where(np.isnan(v), v, np.where(v > 0, v, 0.0))
    if kind == ACT_GELU:
        return 0.5 * v * (1.0 + np.tanh(_GELU_K * (v + 0.044715 * v * v * v)))
    if kind == ACT_SILU:
        with np.errstate(over="ignore"):
            return v / (1.0 + np.exp(-v))
    return v


def f32_to_bf16_bits(f):
    """Round-to-nearest-even, as blas/steel_gemm_test.cc:30-35 writes it."""
    u = np.asarray(f, np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def eps_of(dtype):
    """Unit roundoff used by the reference's tolerance (steel_gemm_test.cc:66-73)."""
    dt = np.dtype(dtype)
    if dt == np.float32:
        return 1e-5
    if dt == np.float16:
        return 1.0 / 1024
    return 1.0 / 128


def gemm(a, b, *, ta=False, tb=False, alpha=1.0, beta=0.0, c=None, bias=None,
         activation=ACT_NONE, out_dtype=None, want_aux=False):
    """Returns (d, aux_or_None, mag) where mag = |alpha| sum|a b| + |beta c|
    (the magnitude the reference's tolerance formula scales by).  Operands
    may carry a leading batch axis; a 2-D operand broadcasts."""
    A = np.asarray(a).astype(np.float64)
    B = np.asarray(b).astype(np.float64)
    if ta:
        A = np.swapaxes(A, -1, -2)
    if tb:
        B = np.swapaxes(B, -1, -2)
    acc = A @ B
    mag = abs(alpha) * (np.abs(A) @ np.abs(B))
    v = alpha * acc
    if beta != 0.0:
        C = np.asarray(c).astype(np.float64)
        v = v + beta * C
        mag = mag + np.abs(beta * C)
    if bias is not None:
        v = v + np.asarray(bias).astype(np.float64)
    out_dtype = out_dtype or np.asarray(a).dtype
    d = act(activation, v).astype(np.float32).astype(out_dtype)
    aux = v.astype(np.float32).astype(out_dtype) if want_aux else None
    return d, aux, mag


def tolerance(want, mag, k, out_dtype):
    """blas/steel_gemm_test.cc:195-196."""
    return eps_of(out_dtype) * np.abs(np.asarray(want, np.float64)) \
        + (1e-5 + 1e-6 * k) * mag + 1e-6


def gemm_work(m, n, k, batch, in_bytes, out_bytes):
    """Cost model of blas/mps_gemm_objc.cc:57-67: max(2 b m n k, 64 * bytes)."""
    flops = 2 * batch * m * n * k
    nbytes = batch * (in_bytes * (m * k + k * n) + out_bytes * m * n)
    return max(flops, 64 * nbytes)


def max_abs_over_rms(got, want):
    """The bf16 acceptance figure: max|got-want| / RMS(want)."""
    got = np.asarray(got).astype(np.float64)
    want = np.asarray(want).astype(np.float64)
    rms = np.sqrt(np.mean(want * want))
    return float(np.max(np.abs(got - want)) / max(rms, 1e-30))
