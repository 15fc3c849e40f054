"""Oracle: one decode step of the Qwen3-shaped decoder (test infrastructure).

Restates examples/llm/qwen3.py:270-390 for T = 1 (one new token per
sequence) on the CPU: embed -> per layer [rms_norm, fused qkv linear, per-head
q/k rms_norm, rope (rotate-half), cache write (K [B,KV,S,D], V [B,KV,D,S]),
grouped-query decode attention with an f32 softmax, o linear + residual,
rms_norm, fused gate_up linear, silu(gate)*up, down linear + residual] ->
final rms_norm -> LM head -> f32 logits.

Activations are bf16 and are rounded wherever the reference casts back to the
activation dtype; reductions are accumulated in float64 and rounded to f32
first.  Linear weights are either a bf16 [out, in] matrix or a dict holding a
quantised one (see `linear`).
"""
import ml_dtypes
import numpy as np

from . import quant
from .rownorm import rms_norm

bf16 = ml_dtypes.bfloat16


def _r(a, dtype=bf16):
    return np.asarray(a).astype(np.float32).astype(dtype)


def linear(x, w):
    """qwen3.py:218-230 (x @ w.T, result in x's dtype).  `w` is a bf16
    [out, in] array, or a dict: {"q4": u32 [N, K/8], "s", "b"} (sequential
    nibbles), {"q4h": u8 [N, G, 32], "s", "b"} (the reference's split-half
    bytes) or {"q": int8 [N, K], "s"}."""
    if isinstance(w, dict):
        if "q4" in w:
            return quant.qmm(x, quant.bl_unpack_int4(w["q4"]), w["s"], w["b"], x.dtype)
        if "q4h" in w:
            q = quant.ref_unpack_int4(w["q4h"])
            q = q.reshape(q.shape[0], -1)
            G = w["q4h"].shape[1]
            return quant.qmm(x, q, np.asarray(w["s"]).reshape(-1, G),
                             np.asarray(w["b"]).reshape(-1, G), x.dtype)
        return quant.qmm(x, w["q"], w["s"], None, x.dtype)
    y = np.asarray(x).astype(np.float64) @ np.asarray(w).astype(np.float64).T
    return y.astype(np.float32).astype(x.dtype)


def rope(x, positions, theta):
    """qwen3.py:300-310.  x [B, H, D] (T = 1 folded away), positions [B]."""
    d = x.shape[-1]
    inv_freq = (1.0 / theta ** (np.arange(0, d, 2, dtype=np.float32) / np.float32(d))).astype(np.float32)
    ang = positions[:, None].astype(np.float32) * inv_freq          # [B, D/2]
    cos = np.cos(ang.astype(np.float64))[:, None, :]
    sin = np.sin(ang.astype(np.float64))[:, None, :]
    x64 = np.asarray(x).astype(np.float64)
    x1, x2 = x64[..., : d // 2], x64[..., d // 2:]
    out = np.concatenate([x1 * cos - x2 * sin, x2 * cos + x1 * sin], axis=-1)
    return out.astype(np.float32).astype(x.dtype)


def silu_mul(gate, up):
    """jax.nn.silu(gate) * up on bf16 arrays (qwen3.py:376): sigmoid, the
    product with gate and the product with up each round to bf16."""
    g32 = np.asarray(gate).astype(np.float32)
    sig = _r(1.0 / (1.0 + np.exp(-g32.astype(np.float64))), gate.dtype)
    act = _r(g32 * sig.astype(np.float32), gate.dtype)
    return _r(act.astype(np.float32) * np.asarray(up).astype(np.float32), gate.dtype)


def attention_decode(q, k_cache, v_cache, n_valid, scale):
    """qwen3.py:322-327.  q [B, KV, G, D]; k_cache [B, KV, S, D]; v_cache
    [B, KV, D, S]; attends slots < n_valid.  Returns [B, KV, G, D] in the
    cache dtype."""
    q64 = np.asarray(q).astype(np.float64)
    k64 = np.asarray(k_cache[:, :, :n_valid]).astype(np.float64)
    v64 = np.asarray(v_cache[..., :n_valid]).astype(np.float64)
    s = np.einsum("bkgd,bksd->bkgs", q64, k64) * scale
    s = s.astype(np.float32).astype(np.float64)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(axis=-1, keepdims=True)
    a = np.einsum("bkgs,bkds->bkgd", p, v64)
    return a.astype(np.float32).astype(v_cache.dtype)


def decode_step(params, tokens, cache, pos, cfg):
    """One token per sequence at absolute position `pos`.  tokens [B] int;
    cache {"k": [L x [B,KV,S,D]], "v": [L x [B,KV,D,S]]} updated IN PLACE.
    cfg: dict with hidden, heads, kv_heads, head_dim, theta, eps.
    Returns f32 logits [B, V]."""
    B = tokens.shape[0]
    H, KV, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    G = H // KV
    eps = cfg["eps"]
    x = np.asarray(params["embed"])[tokens]                            # [B, E] bf16
    positions = np.full((B,), pos, np.int64)
    scale = D ** -0.5
    for li, lp in enumerate(params["layers"]):
        h = rms_norm(x, lp["attn_norm"], eps)
        qkv = linear(h, lp["qkv"])
        q = qkv[:, : H * D].reshape(B, H, D)
        k = qkv[:, H * D:(H + KV) * D].reshape(B, KV, D)
        v = qkv[:, (H + KV) * D:].reshape(B, KV, D)
        q = rope(rms_norm(q, lp["q_norm"], eps), positions, cfg["theta"])
        k = rope(rms_norm(k, lp["k_norm"], eps), positions, cfg["theta"])
        cache["k"][li][:, :, pos, :] = k
        cache["v"][li][:, :, :, pos] = v
        a = attention_decode(q.reshape(B, KV, G, D), cache["k"][li], cache["v"][li],
                             pos + 1, scale).reshape(B, H * D)
        x = _r(x.astype(np.float32) + linear(a, lp["o"]).astype(np.float32), x.dtype)
        h = rms_norm(x, lp["mlp_norm"], eps)
        gu = linear(h, lp["gate_up"])
        inter = gu.shape[-1] // 2
        x = _r(x.astype(np.float32)
               + linear(silu_mul(gu[:, :inter], gu[:, inter:]), lp["down"]).astype(np.float32),
               x.dtype)
    x = rms_norm(x, params["norm"], eps)
    return linear(x, params.get("lm_head", params["embed"])).astype(np.float32)
