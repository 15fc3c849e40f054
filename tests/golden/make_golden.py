"""Generates tests/golden/*.npz from the reference's own Python code.

Run in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It imports examples/llm/qwen3.py from that checkout.  jax is not installed
where this was run, so a NumPy stand-in for the handful of jax / jax.numpy
names that file uses is put into sys.modules first (below).  Everything the
quantisers do is plain NumPy in the reference already, so those vectors are
the reference's bit for bit; the model functions run through the stand-in,
whose semantics are: bf16 arithmetic via ml_dtypes (each op computed in f32
and rounded), f32 reductions by NumPy's pairwise sums, einsum accumulated in
f32 and rounded once.  XLA:CPU's own summation order is not reproduced.
The fixtures are small (a few hundred KB) and are committed with this script.
"""
import importlib.util
import os
import sys
import types

import ml_dtypes
import numpy as np


def _install_jax_stand_in():
    jnp = types.ModuleType("jax.numpy")
    for name in ("concatenate", "sum", "float32", "arange", "broadcast_to", "cos", "sin",
                 "where", "inf", "split", "mean", "argmax", "argsort", "cumsum",
                 "take_along_axis", "int32", "asarray"):
        setattr(jnp, name, getattr(np, name))
    jnp.bfloat16 = ml_dtypes.bfloat16
    jnp.zeros = lambda shape, dtype=np.float32, device=None: np.zeros(shape, dtype)

    def einsum(spec, a, b, preferred_element_type=None):
        out = np.einsum(spec, np.asarray(a).astype(np.float32), np.asarray(b).astype(np.float32))
        return out.astype(preferred_element_type or np.asarray(a).dtype)
    jnp.einsum = einsum

    lax = types.ModuleType("jax.lax")
    lax.rsqrt = lambda v: (1.0 / np.sqrt(v)).astype(np.asarray(v).dtype)

    def dynamic_update_slice(operand, update, start):
        out = np.array(operand, copy=True)
        idx = tuple(slice(int(s), int(s) + n) for s, n in zip(start, update.shape))
        out[idx] = update
        return out
    lax.dynamic_update_slice = dynamic_update_slice
    lax.dynamic_index_in_dim = lambda x, i, axis=0, keepdims=True: \
        np.take(x, [int(i)], axis=axis) if keepdims else np.take(x, int(i), axis=axis)

    nn = types.ModuleType("jax.nn")

    def softmax(x, axis=-1):
        with np.errstate(invalid="ignore"):
            m = np.max(x, axis=axis, keepdims=True)
            e = np.exp(x - m)
            return e / np.sum(e, axis=axis, keepdims=True)
    nn.softmax = softmax

    def silu(x):
        dt = np.asarray(x).dtype
        sig = (1.0 / (1.0 + np.exp(-np.asarray(x).astype(np.float32)))).astype(dt)
        return x * sig
    nn.silu = silu

    jax = types.ModuleType("jax")
    jax.numpy, jax.lax, jax.nn = jnp, lax, nn
    jax.device_put = lambda a, device=None: np.asarray(a)
    sys.modules.update({"jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.nn": nn})


def _load_reference(ref_root):
    _install_jax_stand_in()
    path = os.path.join(ref_root, "examples", "llm", "qwen3.py")
    spec = importlib.util.spec_from_file_location("reference_qwen3", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root):
    ref = _load_reference(ref_root)
    here = os.path.dirname(os.path.abspath(__file__))
    bf16 = ml_dtypes.bfloat16
    rng = np.random.default_rng(1234)

    # --- quantisers and quantised products (qwen3.py:154-267) ----------------
    w = (rng.standard_normal((48, 256), dtype=np.float32) * 0.02).astype(np.float32)
    w[3, 64:128] = 0.0                       # a constant group (scale guard)
    w[5, :64] = np.abs(w[5, :64])            # an all-positive group
    w[7, :64] = -np.abs(w[7, :64])           # an all-negative group
    q8, s8 = ref.quantize_int8(w)
    p4, s4, b4 = ref.quantize_int4(w)
    x = rng.standard_normal((3, 256), dtype=np.float32).astype(bf16)
    w8 = {"q": q8, "s": s8.astype(bf16)}
    w4 = {"q4": p4, "s": s4.astype(bf16), "b": b4.astype(bf16)}
    np.savez_compressed(
        os.path.join(here, "quant_ref.npz"),
        w=w, x=x.view(np.uint16),
        q8=q8, s8=s8, p4=p4, s4=s4, b4=b4,
        deq8=ref.dequantize(w8, bf16).view(np.uint16),
        deq4=ref.dequantize(w4, bf16).view(np.uint16),
        mv8=ref._matvec_int8(x, w8).view(np.uint16),
        mv4=ref._matvec_int4(x, w4).view(np.uint16),
        lin4_rows8=ref.linear(np.concatenate([x, x, x])[:8], w4).view(np.uint16))

    # --- rms_norm, rope, decode attention (qwen3.py:294-331) -----------------
    xr = rng.standard_normal((5, 256), dtype=np.float32).astype(bf16)
    gain = (1.0 + 0.1 * rng.standard_normal((256,), dtype=np.float32)).astype(bf16)
    xr32 = rng.standard_normal((4, 200), dtype=np.float32)
    gain32 = (1.0 + 0.1 * rng.standard_normal((200,), dtype=np.float32)).astype(np.float32)
    xh = rng.standard_normal((2, 1, 4, 64), dtype=np.float32).astype(bf16)
    positions = np.array([[7], [7]])
    B, KV, G, D, S = 2, 2, 2, 64, 24
    q = rng.standard_normal((B, 1, KV, G, D), dtype=np.float32).astype(bf16)
    kc = rng.standard_normal((B, KV, S, D), dtype=np.float32).astype(bf16)
    vc = rng.standard_normal((B, KV, D, S), dtype=np.float32).astype(bf16)
    mask = np.arange(S)[None, :] <= np.array([17])[:, None]
    np.savez_compressed(
        os.path.join(here, "rows_ref.npz"),
        xr=xr.view(np.uint16), gain=gain.view(np.uint16),
        rms_bf16=ref.rms_norm(xr, gain, 1e-6).view(np.uint16),
        xr32=xr32, gain32=gain32, rms_f32=ref.rms_norm(xr32, gain32, 1e-6),
        xh=xh.view(np.uint16), rope=ref.rope(xh, positions, 1e6).view(np.uint16),
        q=q.view(np.uint16), kc=kc.view(np.uint16), vc=vc.view(np.uint16),
        attn=ref.attention(q, kc, vc, mask, D ** -0.5).view(np.uint16))

    # --- a small decoder forward, reference int4 format (qwen3.py:334-390) ----
    cfg = ref.Config(vocab_size=320, hidden_size=128, intermediate_size=256,
                     num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=64, rope_theta=1e6, rms_norm_eps=1e-6,
                     tie_word_embeddings=False)
    E, H, KVh, Dh, I = 128, 4, 2, 64, 256

    def qmat(n, k):
        p, s, b = ref.quantize_int4(rng.standard_normal((n, k), dtype=np.float32) * 0.05)
        return {"q4": p, "s": s.astype(bf16), "b": b.astype(bf16)}

    layers = []
    for _ in range(2):
        layers.append({
            "attn_norm": (1.0 + 0.1 * rng.standard_normal(E, dtype=np.float32)).astype(bf16),
            "qkv": qmat((H + 2 * KVh) * Dh, E),
            "q_norm": (1.0 + 0.1 * rng.standard_normal(Dh, dtype=np.float32)).astype(bf16),
            "k_norm": (1.0 + 0.1 * rng.standard_normal(Dh, dtype=np.float32)).astype(bf16),
            "o": qmat(E, H * Dh),
            "mlp_norm": (1.0 + 0.1 * rng.standard_normal(E, dtype=np.float32)).astype(bf16),
            "gate_up": qmat(2 * I, E),
            "down": qmat(E, I)})
    params = {"embed": (rng.standard_normal((320, E), dtype=np.float32) * 0.05).astype(bf16),
              "layers": layers,
              "norm": (1.0 + 0.1 * rng.standard_normal(E, dtype=np.float32)).astype(bf16),
              "lm_head": (rng.standard_normal((320, E), dtype=np.float32) * 0.05).astype(bf16)}
    Bd, ctx, max_len = 2, 9, 16
    cache = ref.init_cache(cfg, Bd, max_len)
    for li in range(2):
        cache["k"][li][:, :, :ctx] = rng.standard_normal((Bd, KVh, ctx, Dh), dtype=np.float32).astype(bf16)
        cache["v"][li][:, :, :, :ctx] = rng.standard_normal((Bd, KVh, Dh, ctx), dtype=np.float32).astype(bf16)
    tokens = rng.integers(0, 320, size=(Bd, 1))
    out = {"tokens": tokens, "ctx": np.int64(ctx), "max_len": np.int64(max_len)}
    for li in range(2):
        out[f"k_in{li}"] = cache["k"][li].view(np.uint16).copy()
        out[f"v_in{li}"] = cache["v"][li].view(np.uint16).copy()
    logits, new_cache = ref.forward(params, tokens, cache, ctx, cfg, window=max_len)
    out["logits"] = np.asarray(logits, np.float32)
    for li in range(2):
        out[f"k_out{li}"] = new_cache["k"][li].view(np.uint16)
        out[f"v_out{li}"] = new_cache["v"][li].view(np.uint16)
    for name in ("embed", "norm", "lm_head"):
        out[name] = params[name].view(np.uint16)
    for li, lp in enumerate(layers):
        for name, val in lp.items():
            if isinstance(val, dict):
                out[f"l{li}_{name}_q4"] = val["q4"]
                out[f"l{li}_{name}_s"] = val["s"].view(np.uint16)
                out[f"l{li}_{name}_b"] = val["b"].view(np.uint16)
            else:
                out[f"l{li}_{name}"] = val.view(np.uint16)
    np.savez_compressed(os.path.join(here, "decoder_ref.npz"), **out)
    print("golden fixtures written to", here)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <reference checkout>")
    main(sys.argv[1])
