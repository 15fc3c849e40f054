"""Oracle: weight-only quantisation and quantised products (test infrastructure).

Two families:
  * `ref_*`  — the reference's own formats, restated from
    examples/llm/qwen3.py:154-267 (group-wise symmetric int8; MLX-style affine
    int4 packed split-half into uint8).  Pinned by tests/golden/quant_ref.npz.
  * `bl_*`   — the benchmark formats (per-output-channel int8; min/max affine
    int4, eight consecutive-k nibbles per little-endian uint32, bf16 scale and
    bias).  No reference code exists for these: parity unpinned beyond
    round-trip self-consistency.

All weights are stored [out, in] (K contiguous) like the reference
(qwen3.py:102).  bf16 is ml_dtypes.bfloat16 (round-to-nearest-even).
"""
import ml_dtypes
import numpy as np

bf16 = ml_dtypes.bfloat16
GROUP = 64


def to_bf16(a):
    return np.asarray(a, np.float32).astype(bf16)


def bf16_round(a):
    """f32 values rounded to bf16 and widened back (what the device stores)."""
    return to_bf16(a).astype(np.float32)


# ----------------------------------------------------------------------------
# Reference formats (qwen3.py:154-207)
# ----------------------------------------------------------------------------

def ref_quantize_int8(w, group=GROUP):
    """qwen3.py:154-166. q [O, K/g, g] int8, s [O, K/g, 1] f32."""
    w = np.asarray(w, np.float32)
    w = w.reshape(w.shape[0], -1, group)
    s = np.maximum(np.abs(w).max(axis=-1, keepdims=True), 1e-12) / 127.0
    q = np.clip(np.rint(w / s), -127, 127).astype(np.int8)
    return q, s.astype(np.float32)


def ref_quantize_int4(w, group=GROUP):
    """qwen3.py:169-196. packed [O, K/g, g/2] uint8 (low nibble = element j,
    high nibble = element j + g/2), s and b [O, K/g, 1] f32.  The grid is
    anchored at the group's largest-magnitude edge and stretched so zero
    falls on it; the step may be negative."""
    w = np.asarray(w, np.float32)
    w = w.reshape(w.shape[0], -1, group)
    lo, hi = w.min(axis=-1, keepdims=True), w.max(axis=-1, keepdims=True)
    neg = np.abs(lo) > np.abs(hi)
    s = np.maximum(hi - lo, 1e-12) / 15.0
    s = np.where(neg, s, -s)
    edge = np.where(neg, lo, hi)
    q0 = np.rint(edge / s)
    s = np.where(q0 != 0, edge / np.where(q0 != 0, q0, 1), s)
    b = np.where(q0 == 0, 0.0, edge)
    q = np.clip(np.rint((w - b) / s), 0, 15).astype(np.uint8)
    half = group // 2
    return (q[..., :half] | (q[..., half:] << 4)), s.astype(np.float32), b.astype(np.float32)


def ref_unpack_int4(p):
    """[O, G, g/2] uint8 -> [O, G, g] uint8 in k order (qwen3.py:203)."""
    return np.concatenate([p & 0xF, p >> 4], axis=-1)


def ref_dequantize_int4(p, s, b, dtype=bf16):
    """qwen3.py:199-207: computed in the activation dtype, one rounding per op."""
    q = ref_unpack_int4(p).astype(dtype)
    wd = q * np.asarray(s).astype(dtype) + np.asarray(b).astype(dtype)
    return wd.reshape(wd.shape[0], -1)


def ref_dequantize_int8(q, s, dtype=bf16):
    wd = q.astype(dtype) * np.asarray(s).astype(dtype)
    return wd.reshape(wd.shape[0], -1)


def ref_matvec_int8(x, q, s):
    """qwen3.py:233-240: all in f32, one reduction over (group, element);
    result cast to x's dtype."""
    O, G, g = q.shape
    xg = np.asarray(x).reshape(-1, 1, G, g).astype(np.float32)
    t = xg * q.astype(np.float32) * np.asarray(s).astype(np.float32)
    return t.sum(axis=(2, 3), dtype=np.float64).astype(np.float32) \
        .reshape(*x.shape[:-1], O).astype(x.dtype)


def ref_matvec_int4(x, p, s, b):
    """qwen3.py:243-267: per byte (x_lo*lo + x_hi*hi)*s + (x_lo+x_hi)*b in f32,
    summed over (group, byte); result cast to x's dtype."""
    O, G, half = p.shape
    lead = x.shape[:-1]
    xg = np.asarray(x).reshape(-1, 1, G, 2, half).astype(np.float32)
    lo = (p & 0xF).astype(np.float32)
    hi = (p >> 4).astype(np.float32)
    xlo, xhi = xg[:, :, :, 0], xg[:, :, :, 1]
    s = np.asarray(s).astype(np.float32)
    b = np.asarray(b).astype(np.float32)
    t = (xlo * lo + xhi * hi) * s + (xlo + xhi) * b
    return t.sum(axis=(2, 3), dtype=np.float64).astype(np.float32) \
        .reshape(*lead, O).astype(x.dtype)


# ----------------------------------------------------------------------------
# Benchmark formats (no reference code; parity unpinned)
# ----------------------------------------------------------------------------

def bl_quantize_int8(w, group=None):
    """Symmetric int8, one scale per output channel (group=None -> whole row)
    or per `group` inputs.  w [N, K] f32.  q is computed with the f32 scale
    and the scale is then stored as bf16 (what the reference's loader does,
    qwen3.py:113,127).  Returns q [N, K] int8, s [N, K/group] bf16."""
    w = np.asarray(w, np.float32)
    N, K = w.shape
    g = K if group is None else group
    wg = w.reshape(N, K // g, g)
    s = np.maximum(np.abs(wg).max(axis=-1, keepdims=True), 1e-12) / np.float32(127.0)
    q = np.clip(np.rint(wg / s), -127, 127).astype(np.int8).reshape(N, K)
    return q, to_bf16(s.reshape(N, K // g))


def bl_quantize_int4(w, group=GROUP):
    """Affine int4: per group of `group` inputs scale=(max-min)/15, bias=min;
    q=clip(rint((w-bias)/scale),0,15) with the f32 scale/bias, which are then
    stored as bf16.  Packed eight consecutive-k nibbles per uint32, element
    k=8i+j at bits 4j..4j+3.  w [N, K] f32.
    Returns packed [N, K/8] uint32, scale [N, K/group] bf16, bias likewise."""
    w = np.asarray(w, np.float32)
    N, K = w.shape
    wg = w.reshape(N, K // group, group)
    lo, hi = wg.min(axis=-1, keepdims=True), wg.max(axis=-1, keepdims=True)
    s = np.maximum(hi - lo, np.float32(1e-12)) / np.float32(15.0)
    q = np.clip(np.rint((wg - lo) / s), 0, 15).astype(np.uint32).reshape(N, K)
    return bl_pack_int4(q), to_bf16(s.reshape(N, -1)), to_bf16(lo.reshape(N, -1))


def bl_pack_int4(q):
    """[N, K] values 0..15 -> [N, K/8] uint32, k=8i+j at bits 4j..4j+3."""
    q = np.asarray(q).astype(np.uint32)
    N, K = q.shape
    q8 = q.reshape(N, K // 8, 8)
    out = np.zeros((N, K // 8), np.uint32)
    for j in range(8):
        out |= q8[:, :, j] << np.uint32(4 * j)
    return out


def bl_unpack_int4(packed):
    """[N, K/8] uint32 -> [N, K] uint8 in k order."""
    packed = np.asarray(packed, np.uint32)
    N, W = packed.shape
    out = np.empty((N, W, 8), np.uint8)
    for j in range(8):
        out[:, :, j] = (packed >> np.uint32(4 * j)) & np.uint32(0xF)
    return out.reshape(N, W * 8)


def split_half_to_seq(p):
    """The reference's split-half uint8 layout [O, G, g/2] re-expressed as the
    sequential uint32 layout [O, K/8] (same q values, k order)."""
    q = ref_unpack_int4(p)
    return bl_pack_int4(q.reshape(q.shape[0], -1))


def dequant_f32(q_values, scale, bias=None, group=GROUP):
    """The bit-exactness target: w = q*s (+ b) evaluated in f32 from the
    bf16-stored s, b, one rounding per operation (multiply, then add; no fma).
    q_values [N, K] integer; scale/bias [N, K/group]."""
    q = np.asarray(q_values).astype(np.float32)
    N, K = q.shape
    g = K // np.asarray(scale).shape[1]
    s = np.repeat(np.asarray(scale).astype(np.float32), g, axis=1)
    w = q * s
    if bias is not None:
        w = w + np.repeat(np.asarray(bias).astype(np.float32), g, axis=1)
    return w.astype(np.float32)


def qmm(x, q_values, scale, bias=None, out_dtype=bf16):
    """out[M, N] = x[M, K] . dequant(W)[N, K]^T with f64 accumulation of the f32
    dequantised weights (the 'true answer for the rounded inputs'), rounded to
    f32 and then once to `out_dtype`."""
    w = dequant_f32(q_values, scale, bias).astype(np.float64)
    y = np.asarray(x).astype(np.float64) @ w.T
    return y.astype(np.float32).astype(out_dtype)
