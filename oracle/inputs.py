"""Seeded synthetic inputs for the five benchmark configurations (test
infrastructure).  Generator: numpy default_rng(seed).standard_normal in f32,
drawn in the order listed in each function, then scaled and cast.

Reading of "N(0, a)": `a` is the standard deviation, except the config-1
weight N(0, 1/1024) where 1/1024 is the variance (sigma = 1/32), so that
x @ W has unit variance.  No public dataset stands behind any of these.
"""
import ml_dtypes
import numpy as np

from . import quant

bf16 = ml_dtypes.bfloat16

# Qwen3-8B projection shapes as (K, N)
QWEN3_8B_SHAPES = {"q/o": (4096, 4096), "k/v": (4096, 1024),
                   "gate/up": (4096, 12288), "down": (12288, 4096)}


def _n(rng, shape, sigma=1.0):
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma)).astype(np.float32)


def config1(m=512, k=1024, n=1024, seed=0):
    """f32 block: x[m,k] @ W[k,n] + b[n], then RMSNorm(eps 1e-6, gain[n])."""
    rng = np.random.default_rng(seed)
    x = _n(rng, (m, k))
    w = _n(rng, (k, n), 1.0 / 32.0)
    b = _n(rng, (n,), 0.01)
    gain = (1.0 + 0.1 * rng.standard_normal((n,), dtype=np.float32)).astype(np.float32)
    return x, w, b, gain


def config2(m, k=4096, n=4096, seed=1):
    """bf16 A[m,k], B[k,n], bias[n] for D = silu(A @ B + bias)."""
    rng = np.random.default_rng(seed)
    a = _n(rng, (m, k)).astype(bf16)
    b = _n(rng, (k, n), 0.02).astype(bf16)
    bias = _n(rng, (n,), 0.01).astype(bf16)
    return a, b, bias


def config3(m, k, n, seed=2):
    """int8 per-output-channel weights [n, k] + bf16 activations [m, k]."""
    rng = np.random.default_rng(seed)
    w = _n(rng, (n, k), 0.02)
    x = _n(rng, (m, k)).astype(bf16)
    q, s = quant.bl_quantize_int8(w)
    return x, q, s, w


def config4(m, k, n, seed=3, group=64):
    """int4 group-wise affine weights [n, k] + bf16 activations [m, k]."""
    rng = np.random.default_rng(seed)
    w = _n(rng, (n, k), 0.02)
    x = _n(rng, (m, k)).astype(bf16)
    packed, s, b = quant.bl_quantize_int4(w, group)
    return x, packed, s, b, w


def config4_rows(m, hidden=4096, heads=32, ctx=2048, seed=3):
    """The row passes that follow each config-4 product: a bf16 RMSNorm input
    [m, hidden] with gain 1 + 0.1 N(0,1), and f32 softmax logits
    [m*heads, ctx] ~ N(0, 3)."""
    rng = np.random.default_rng(seed + 1000)
    h = _n(rng, (m, hidden)).astype(bf16)
    gain = (1.0 + 0.1 * rng.standard_normal((hidden,), dtype=np.float32)).astype(bf16)
    logits = _n(rng, (m * heads, ctx), 3.0)
    return h, gain, logits


def decoder_config(layers=36, hidden=4096, heads=32, kv_heads=8, head_dim=128,
                   inter=12288, vocab=151936, theta=1e6, eps=1e-6):
    return dict(layers=layers, hidden=hidden, heads=heads, kv_heads=kv_heads,
                head_dim=head_dim, inter=inter, vocab=vocab, theta=theta, eps=eps)


def config5(cfg, batch, ctx, seed=4, max_len=None, group=64):
    """Random-init int4-g64 decoder parameters, a KV cache holding `ctx` prior
    tokens ~N(0,1), and one token id per sequence.  Sizes come from `cfg`
    (decoder_config); the full Qwen3-8B shape is only generated on the GPU
    side, this NumPy version serves the reduced parity cases."""
    rng = np.random.default_rng(seed)
    E, H, KV, D = cfg["hidden"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    I, V = cfg["inter"], cfg["vocab"]
    S = max_len or (ctx + 1)

    def qmat(n, k):
        packed, s, b = quant.bl_quantize_int4(_n(rng, (n, k), 0.02), group)
        return {"q4": packed, "s": s, "b": b}

    layers = []
    for _ in range(cfg["layers"]):
        layers.append({
            "attn_norm": np.ones((E,), bf16),
            "qkv": qmat((H + 2 * KV) * D, E),
            "q_norm": np.ones((D,), bf16),
            "k_norm": np.ones((D,), bf16),
            "o": qmat(E, H * D),
            "mlp_norm": np.ones((E,), bf16),
            "gate_up": qmat(2 * I, E),
            "down": qmat(E, I),
        })
    params = {"embed": _n(rng, (V, E), 0.02).astype(bf16), "layers": layers,
              "norm": np.ones((E,), bf16),
              "lm_head": _n(rng, (V, E), 0.02).astype(bf16)}
    cache = {"k": [], "v": []}
    for _ in range(cfg["layers"]):
        k = np.zeros((batch, KV, S, D), bf16)
        v = np.zeros((batch, KV, D, S), bf16)
        k[:, :, :ctx] = _n(rng, (batch, KV, ctx, D)).astype(bf16)
        v[:, :, :, :ctx] = _n(rng, (batch, KV, D, ctx)).astype(bf16)
        cache["k"].append(k)
        cache["v"].append(v)
    tokens = rng.integers(0, V, size=(batch,), dtype=np.int64)
    return params, cache, tokens
