"""Model-level mirror of examples/llm/qwen3.py for the decode path: the same
function names and argument meaning (quantize_int4 / quantize_int8 /
dequantize / linear / rms_norm / init_cache / forward for T = 1), served by
libb200graft.so.  Weights are dicts of torch CUDA tensors:

    {"q4": int32 [N, K/8]  (uint32 words, k = 8i+j at bits 4j..4j+3), "s": bf16 [N, K/64], "b": bf16 [N, K/64]}
    {"q4h": uint8 [N, K/64, 32] (the reference's split-half bytes),   "s": ..., "b": ...}
    {"q": int8 [N, K], "s": bf16 [N, K/group]}          group == K: per output channel
or a plain bf16 [N, K] tensor.  Nothing here computes on the host.
"""
import ctypes as C

from . import _lib
from .context import default_context
from .rows import rms_norm  # noqa: F401  (qwen3.py:294-297)

GROUP = 64
ROWS_MAX = 32  # the streaming kernel's row limit (the reference's is 4, qwen3.py:215)


def _torch():
    import torch
    return torch


def quantize_int4(w, group=GROUP, ctx=None):
    """≙ quantize_int4 (qwen3.py:169-196) in the benchmark's min/max variant,
    on the device. w: f32 or bf16 [N, K]."""
    torch = _torch()
    ctx = ctx or default_context(w.device.index or 0)
    N, K = w.shape
    w = w.contiguous()
    q = torch.empty((N, K // 8), dtype=torch.int32, device=w.device)
    s = torch.empty((N, K // group), dtype=torch.bfloat16, device=w.device)
    b = torch.empty_like(s)
    _lib.check(_lib.lib().b200_quantize(ctx.handle, _lib.current_stream(), 4, group, _lib.ptr(w),
                                        _lib.dtype_code(w.dtype), _lib.ptr(q), _lib.ptr(s), _lib.ptr(b), N, K))
    return {"q4": q, "s": s, "b": b}


def quantize_int8(w, group=None, ctx=None):
    """≙ quantize_int8 (qwen3.py:154-166); group None = one scale per output channel."""
    torch = _torch()
    ctx = ctx or default_context(w.device.index or 0)
    N, K = w.shape
    g = K if group is None else group
    w = w.contiguous()
    q = torch.empty((N, K), dtype=torch.int8, device=w.device)
    s = torch.empty((N, K // g), dtype=torch.bfloat16, device=w.device)
    _lib.check(_lib.lib().b200_quantize(ctx.handle, _lib.current_stream(), 8, g, _lib.ptr(w),
                                        _lib.dtype_code(w.dtype), _lib.ptr(q), _lib.ptr(s), None, N, K))
    return {"q": q, "s": s}


def _describe(w):
    """(bits, group, nibble_order, q, scale, bias, N, K) of a weight."""
    if isinstance(w, dict):
        if "q4" in w:
            N, W = w["q4"].shape
            return 4, 64, 0, w["q4"], w["s"], w["b"], N, W * 8
        if "q4h" in w:
            N, G, _ = w["q4h"].shape
            return 4, 64, 1, w["q4h"], w["s"], w["b"], N, G * 64
        N, K = w["q"].shape
        return 8, K // w["s"].shape[1], 0, w["q"], w["s"], None, N, K
    N, K = w.shape
    return 16, 0, 0, w, None, None, N, K


def dequantize(w, dtype=None, ctx=None):
    """≙ dequantize (qwen3.py:199-207): the [out, in] matrix of a quantised
    weight, f32 (one rounding per operation) or bf16."""
    torch = _torch()
    bits, group, order, q, s, b, N, K = _describe(w)
    ctx = ctx or default_context(q.device.index or 0)
    dtype = dtype or torch.float32
    out = torch.empty((N, K), dtype=dtype, device=q.device)
    _lib.check(_lib.lib().b200_dequantize(ctx.handle, _lib.current_stream(), bits, group, order, _lib.ptr(q),
                                          _lib.ptr(s), _lib.ptr(b), _lib.ptr(out), N, K, _lib.dtype_code(dtype)))
    return out


def interleave_gate_up(w, ctx=None):
    """A quantised [gate | up] projection with its rows rearranged for linear(..., silu_pair=True):
    every 16 consecutive rows hold 8 gate rows, then the 8 up rows of the same outputs."""
    torch = _torch()
    first = next(iter(w.values()))
    ctx = ctx or default_context(first.device.index or 0)
    out = {}
    for k, v in w.items():
        v = v.contiguous()
        rows = v.shape[0]
        o = torch.empty_like(v)
        _lib.check(_lib.lib().b200_interleave_gate_up(ctx.handle, _lib.current_stream(), _lib.ptr(v), _lib.ptr(o), rows // 2,
                                                     v.numel() // rows * v.element_size()))
        out[k] = o
    return out


def linear(x, w, residual=None, out_f32=False, rms_gain=None, eps=1e-6, silu_mul=False, silu_pair=False, ctx=None,
           stream=None):
    """≙ linear (qwen3.py:218-230): x @ w.T for an [out, in] weight, bf16 or
    quantised, up to ROWS_MAX rows; result in x's dtype (bf16).  `residual`
    fuses the x + linear(...) of the decoder layer; out_f32 gives the LM head's
    f32 logits.  rms_gain fuses linear(rms_norm(x, rms_gain, eps), w) (up to 8
    rows); silu_mul fuses linear(silu(gate) * up, w) for x = [gate | up]."""
    torch = _torch()
    ctx = ctx or default_context(x.device.index or 0)
    bits, group, order, q, s, b, N, K = _describe(w)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, 2 * K if silu_mul else K)
    M = x2.shape[0]
    n_out = N // 2 if silu_pair else N   # silu_pair: w from interleave_gate_up; the result is silu(gate) * up
    out = torch.empty((M, n_out), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    p = _lib.QmmParamsC()
    p.bits, p.group, p.nibble_order = bits, group, order
    p.epilogue = _lib.QMM_OUT_F32 if out_f32 else (_lib.QMM_ADD_RESIDUAL if residual is not None else _lib.QMM_OUT_BF16)
    if silu_pair:
        p.epilogue = _lib.QMM_OUT_SILU_PAIR
    p.x, p.q = x2.data_ptr(), q.data_ptr()
    p.scale = s.data_ptr() if s is not None else None
    p.bias = b.data_ptr() if b is not None else None
    p.residual = residual.data_ptr() if residual is not None else None
    p.out = out.data_ptr()
    p.M, p.N, p.K = M, N, K
    p.ldx, p.ldo = x2.stride(0) if M > 0 else 0, n_out
    if rms_gain is not None:
        p.prologue, p.eps, p.prologue_gain = _lib.QMM_PRO_RMSNORM, eps, rms_gain.data_ptr()
    elif silu_mul:
        p.prologue = _lib.QMM_PRO_SILU_MUL
    _lib.check(_lib.lib().b200_qmm_run(ctx.handle, stream or _lib.current_stream(), C.byref(p)))
    return out.reshape(*lead, n_out)


def qmm_plan(M, N, K, bits=4, group=64):
    """(rows per CTA, CTAs along K, batch blocks) the library would use."""
    p = _lib.QmmParamsC()
    p.bits, p.group, p.M, p.N, p.K = bits, group, M, N, K
    p.x = p.q = p.scale = p.bias = p.out = 16  # non-null placeholders; nothing is dereferenced
    r, s, m = C.c_int(), C.c_int(), C.c_int()
    _lib.check(_lib.lib().b200_qmm_plan(C.byref(p), C.byref(r), C.byref(s), C.byref(m)))
    return r.value, s.value, m.value


def sample(logits, uniform=None, *, temperature=0.0, top_k=0, top_p=1.0, ctx=None, stream=None):
    """≙ sample (qwen3.py:395-418): next token int32 [B] from f32 logits [B, V] on the device;
    temperature 0 is greedy.  `uniform` (f32 [B] in [0, 1), device) replaces the reference's
    PRNG key: the categorical draw is the inverse CDF at that number."""
    torch = _torch()
    ctx = ctx or default_context(logits.device.index or 0)
    B, V = logits.shape
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    _lib.check(_lib.lib().b200_sample(ctx.handle, stream or _lib.current_stream(), _lib.ptr(logits.contiguous()), B, V,
                                      float(temperature), int(top_k), float(top_p), _lib.ptr(uniform), _lib.ptr(out)))
    return out


def init_cache(cfg, batch, max_len, device="cuda"):
    """≙ init_cache (qwen3.py:279-291): per-layer K [B, KV, S, D] and V [B, KV, D, S]."""
    torch = _torch()
    k = (batch, cfg["kv_heads"], max_len, cfg["head_dim"])
    v = (batch, cfg["kv_heads"], cfg["head_dim"], max_len)
    return {"k": [torch.zeros(k, dtype=torch.bfloat16, device=device) for _ in range(cfg["layers"])],
            "v": [torch.zeros(v, dtype=torch.bfloat16, device=device) for _ in range(cfg["layers"])]}


class Decoder:
    """One-token decode step (≙ forward with T = 1, qwen3.py:334-390, driven like
    generate.Engine.step, examples/llm/generate.py:146-148).  `params` follows
    the reference's pytree: {"embed", "layers": [{"attn_norm", "qkv", "q_norm",
    "k_norm", "o", "mlp_norm", "gate_up", "down"}], "norm", "lm_head"} with int4
    ("q4") projections; `cache` comes from init_cache.  With `tp` the params and
    cache hold this rank's shard and cfg the local head / intermediate / vocab
    counts (see parallel.shard_params)."""

    def __init__(self, params, cache, cfg, max_batch, ctx=None, tp=None):
        self.ctx = ctx or default_context(params["embed"].device.index or 0)
        self.cfg, self.params, self.cache, self.tp = cfg, params, cache, tp
        L = cfg["layers"]
        max_len = cache["k"][0].shape[2]
        cc = _lib.DecoderConfigC(L, cfg["hidden"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["inter"],
                                 cfg["vocab"], max_len, cfg["theta"], cfg["eps"], max_batch)
        layers = (_lib.DecoderLayerC * L)()
        for i, lp in enumerate(params["layers"]):
            def qw(w):
                return _lib.QWeightC(w["q4"].data_ptr(), w["s"].data_ptr(), w["b"].data_ptr())
            layers[i] = _lib.DecoderLayerC(lp["attn_norm"].data_ptr(), qw(lp["qkv"]), lp["q_norm"].data_ptr(),
                                           lp["k_norm"].data_ptr(), qw(lp["o"]), lp["mlp_norm"].data_ptr(),
                                           qw(lp["gate_up"]), qw(lp["down"]), cache["k"][i].data_ptr(),
                                           cache["v"][i].data_ptr())
        handle = C.c_void_p()
        _lib.check(_lib.lib().b200_decoder_create(self.ctx.handle, C.byref(cc), layers, params["embed"].data_ptr(),
                                                  params["norm"].data_ptr(), params["lm_head"].data_ptr(),
                                                  tp.handle if tp is not None else None, C.byref(handle)))
        self.handle = handle
        self.world = tp.world if tp is not None else 1

    def step(self, tokens, pos, logits=None, stream=None):
        """tokens int32 [B] (device), pos int32 [1] (device). Returns f32 logits
        [B, V]; with tp [world, B, V/world] (rank-major)."""
        torch = _torch()
        B = tokens.shape[0]
        if logits is None:
            shape = (B, self.cfg["vocab"]) if self.world == 1 else (self.world, B, self.cfg["vocab"])
            logits = torch.empty(shape, dtype=torch.float32, device=tokens.device)
        _lib.check(_lib.lib().b200_decoder_step(self.handle, stream or _lib.current_stream(), _lib.ptr(tokens),
                                                _lib.ptr(pos), _lib.ptr(logits), B))
        return logits

    def launches_per_step(self, batch):
        """1 where the whole step is the single persistent kernel, else the graph's kernel count."""
        return _lib.lib().b200_decoder_launches_per_step(self.handle, batch)

    def graphs_built(self):
        """CUDA graphs captured so far (0 while every step took the single kernel)."""
        return _lib.lib().b200_decoder_graphs_built(self.handle)

    def trace(self, enable=True):
        """Per-stage time stamps inside the single-kernel step (b200_decoder_trace)."""
        _lib.check(_lib.lib().b200_decoder_trace(self.handle, 1 if enable else 0))

    def read_trace(self):
        """(stamps uint64 [ctas, stages, 4] in ns, stage kinds int32 [stages]) of the last
        traced step; synchronise the stream first."""
        import numpy as np
        ctas, stages = C.c_int32(), C.c_int32()
        _lib.check(_lib.lib().b200_decoder_trace_read(self.handle, None, 0, C.byref(ctas), C.byref(stages), None))
        out = np.zeros((ctas.value, stages.value, 4), np.uint64)
        kinds = np.zeros(stages.value, np.int32)
        _lib.check(_lib.lib().b200_decoder_trace_read(self.handle, out.ctypes.data_as(C.c_void_p), out.size,
                                                      C.byref(ctas), C.byref(stages), kinds.ctypes.data_as(C.c_void_p)))
        return out, kinds

    def close(self):
        if self.handle:
            _lib.lib().b200_decoder_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
