"""Checkpoint loading (≙ Config.from_json, read_safetensors, load_params of
examples/llm/qwen3.py:24-148): a dense Qwen3 checkpoint directory (config.json +
*.safetensors) to the parameter pytree qwen3.Decoder takes, quantised at load time ON THE
DEVICE in blocks of rows.

Differences from the reference, on purpose: tensors land in torch CUDA tensors instead of
JAX arrays; quantisation runs on the GPU (b200_quantize_int4_ref reproduces the
reference's NumPy quantiser bit for bit, b200_quantize bits 8 / group 64 its int8 one);
the embedding and the LM head stay bf16 (the decoder kernel takes a bf16 table and head);
`layout="seq"` (default) repacks the int4 bytes into the sequential uint32 words the
decoder streams, `layout="ref"` keeps the reference's split-half bytes ("q4h", accepted by
qwen3.linear)."""
import dataclasses
import glob
import json
import mmap
import os
import struct

import ml_dtypes
import numpy as np

from . import _lib
from .context import default_context


@dataclasses.dataclass(frozen=True)
class Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool

    @classmethod
    def from_json(cls, path):
        """A dense Qwen3 config; refuses what the reference refuses (qwen3.py:37-52): other
        model types, rope scaling, quantised checkpoints."""
        with open(path) as f:
            d = json.load(f)
        if d.get("model_type") != "qwen3":
            raise ValueError(f"not a dense Qwen3 checkpoint: model_type {d.get('model_type')!r}")
        if d.get("rope_scaling"):
            raise ValueError(f"rope_scaling {d['rope_scaling']!r} is not supported")
        if d.get("quantization_config"):
            raise ValueError("quantized checkpoints (e.g. FP8) are not supported; use the bf16 one and quant=")
        return cls(**{k.name: d[k.name] for k in dataclasses.fields(cls)})

    def decoder_cfg(self):
        """The dict qwen3.Decoder takes."""
        return dict(layers=self.num_hidden_layers, hidden=self.hidden_size, heads=self.num_attention_heads,
                    kv_heads=self.num_key_value_heads, head_dim=self.head_dim, inter=self.intermediate_size,
                    vocab=self.vocab_size, theta=self.rope_theta, eps=self.rms_norm_eps)


_DTYPES = {"BF16": ml_dtypes.bfloat16, "F16": np.float16, "F32": np.float32}


def read_safetensors(path):
    """{name: np.ndarray} backed by an mmap of the file (≙ qwen3.py:75-98): 8-byte
    little-endian header length, a JSON header of {name: {dtype, shape, data_offsets}},
    then the raw data."""
    with open(path, "rb") as f:
        buf = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    (n,) = struct.unpack("<Q", buf[:8])
    header = json.loads(buf[8:8 + n])
    header.pop("__metadata__", None)
    out = {}
    for name, info in header.items():
        start, _ = info["data_offsets"]
        if info["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name} has dtype {info['dtype']}; only {', '.join(_DTYPES)} checkpoints "
                             "are supported")
        out[name] = np.frombuffer(buf, dtype=_DTYPES[info["dtype"]], count=int(np.prod(info["shape"])),
                                  offset=8 + n + start).reshape(info["shape"])
    return out


def _to_device(a, device):
    """NumPy (bf16 / f16 / f32) -> torch tensor on the device, bit for bit."""
    import torch
    a = np.ascontiguousarray(a)
    if a.dtype == ml_dtypes.bfloat16:
        return torch.from_numpy(a.view(np.int16)).to(device).view(torch.bfloat16)
    return torch.from_numpy(a).to(device)


def quantize_int4_ref(w, layout="seq", ctx=None):
    """The reference's quantize_int4 on the device.  w: CUDA tensor f32 / bf16 [N, K]."""
    import torch
    ctx = ctx or default_context(w.device.index or 0)
    N, K = w.shape
    w = w.contiguous()
    q = torch.empty((N, K // 64, 32), dtype=torch.uint8, device=w.device)
    s = torch.empty((N, K // 64), dtype=torch.bfloat16, device=w.device)
    b = torch.empty_like(s)
    stream = _lib.current_stream()
    _lib.check(_lib.lib().b200_quantize_int4_ref(ctx.handle, stream, _lib.ptr(w), _lib.dtype_code(w.dtype), _lib.ptr(q),
                                                 _lib.ptr(s), _lib.ptr(b), N, K))
    if layout == "ref":
        return {"q4h": q, "s": s, "b": b}
    seq = torch.empty((N, K // 8), dtype=torch.int32, device=w.device)
    _lib.check(_lib.lib().b200_repack_int4(ctx.handle, stream, _lib.ptr(q), _lib.ptr(seq), N, K))
    return {"q4": seq, "s": s, "b": b}


def load_params(path, cfg, device="cuda", quant="int4", layout="seq", ctx=None, block_rows=8192):
    """Parameters as the reference's pytree (qwen3.py:101-148): a list of per-layer dicts, the
    q/k/v projections concatenated into `qkv`, gate/up into `gate_up`, matrices [out, in].
    quant: None (bf16), "int8" (q int8 [N, K], s bf16 [N, K/64]) or "int4"."""
    import torch
    from . import qwen3
    t = {}
    for f in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
        t.update(read_safetensors(f))
    put = lambda a: _to_device(np.asarray(a).astype(ml_dtypes.bfloat16), device)

    def mat(*names):
        if quant is None:
            return put(np.concatenate([t[n] for n in names]) if len(names) > 1 else t[names[0]])
        if quant not in ("int8", "int4"):
            raise ValueError(f"unknown quant {quant!r}")
        parts = []
        for n in names:   # in blocks of rows: a whole matrix in f32 on the way would take GBs
            w = t[n]
            for i in range(0, w.shape[0], block_rows):
                wd = _to_device(w[i:i + block_rows], device).float()
                parts.append(quantize_int4_ref(wd, layout, ctx) if quant == "int4" else qwen3.quantize_int8(wd, 64, ctx))
        return {k: torch.cat([p[k] for p in parts]) for k in parts[0]}

    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        w = lambda n: p + n + ".weight"
        layers.append({
            "attn_norm": put(t[w("input_layernorm")]),
            "qkv": mat(w("self_attn.q_proj"), w("self_attn.k_proj"), w("self_attn.v_proj")),
            "q_norm": put(t[w("self_attn.q_norm")]),
            "k_norm": put(t[w("self_attn.k_norm")]),
            "o": mat(w("self_attn.o_proj")),
            "mlp_norm": put(t[w("post_attention_layernorm")]),
            "gate_up": mat(w("mlp.gate_proj"), w("mlp.up_proj")),
            "down": mat(w("mlp.down_proj")),
        })
    params = {"embed": put(t["model.embed_tokens.weight"]), "layers": layers, "norm": put(t["model.norm.weight"])}
    params["lm_head"] = params["embed"] if cfg.tie_word_embeddings else put(t["lm_head.weight"])
    return params
