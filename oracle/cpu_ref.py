"""ctypes loader of the C restatement (oracle/cpu_ref.c): test / benchmark
infrastructure, used as the timed CPU baseline and as a cross-check of the
NumPy oracle."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


class Cfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("layers", "hidden", "heads", "kv_heads", "head_dim", "inter", "vocab",
                                         "max_len")] + [("theta", C.c_float), ("eps", C.c_float)]


class Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "attn_norm", "qkv_q", "qkv_s", "qkv_b", "q_norm", "k_norm", "o_q", "o_s", "o_b", "mlp_norm",
        "gu_q", "gu_s", "gu_b", "down_q", "down_s", "down_b", "k_cache", "v_cache")]


_lib = None


def lib():
    global _lib
    if _lib is None:
        flags = ""
        try:
            with open("/proc/cpuinfo") as f:
                flags = f.read()
        except OSError:
            pass
        name = "cpu_ref_avx2.so" if (" avx2" in flags and " fma" in flags) else "cpu_ref_base.so"
        path = os.path.join(HERE, "_build", name)
        if not os.path.exists(path):
            from . import build as _b
            _b.build()
        _lib = C.CDLL(path)
        _lib.oracle_threads.restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def threads():
    return lib().oracle_threads()


def set_threads(n):
    """Use n threads from now on, whatever OMP_NUM_THREADS said at load time."""
    lib().oracle_set_threads(int(n))


def qmv_int4(x, q, s, b):
    """x bf16 [M,K]; q uint32 [N,K/8]; s,b bf16 [N,K/64] -> f32 [M,N] (unrounded)."""
    M, K = x.shape
    N = q.shape[0]
    out = np.empty((M, N), np.float32)
    lib().oracle_qmv_int4(_p(np.ascontiguousarray(x)), _p(np.ascontiguousarray(q)), _p(np.ascontiguousarray(s)),
                          _p(np.ascontiguousarray(b)), _p(out), M, N, K)
    return out


def qmv_int8(x, q, s):
    M, K = x.shape
    N = q.shape[0]
    out = np.empty((M, N), np.float32)
    lib().oracle_qmv_int8(_p(np.ascontiguousarray(x)), _p(np.ascontiguousarray(q)), _p(np.ascontiguousarray(s)),
                          _p(out), M, N, K, K // s.shape[1])
    return out


def mv_bf16(x, w):
    M, K = x.shape
    N = w.shape[0]
    out = np.empty((M, N), np.float32)
    lib().oracle_mv_bf16(_p(np.ascontiguousarray(x)), _p(np.ascontiguousarray(w)), _p(out), M, N, K)
    return out


def gemm_f32(a, b, bias):
    M, K = a.shape
    N = b.shape[1]
    out = np.empty((M, N), np.float32)
    lib().oracle_gemm_f32(_p(a), _p(b), _p(bias) if bias is not None else None, _p(out), M, N, K)
    return out


def rms_norm_f32(x, w, eps):
    y = np.empty_like(x)
    lib().oracle_rms_norm_f32(_p(x), _p(w), _p(y), x.shape[0], x.shape[1], C.c_float(eps))
    return y


def softmax_f32(x):
    y = np.empty_like(x)
    lib().oracle_softmax_f32(_p(x), _p(y), x.shape[0], x.shape[1])
    return y


def layer_norm_f32(x, eps=1e-5):
    y = np.empty_like(x)
    lib().oracle_layer_norm_f32(_p(x), _p(y), x.shape[0], x.shape[1], C.c_float(eps))
    return y


def decode_step(params, tokens, cache, pos, cfg, run_layers=None, run_vocab=None):
    """Same arguments as oracle.decoder.decode_step (int4 'q4' projections);
    updates the cache in place; returns f32 logits [B, run_vocab]."""
    max_len = cache["k"][0].shape[2]
    c = Cfg(cfg["layers"], cfg["hidden"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["inter"],
            cfg["vocab"], max_len, cfg["theta"], cfg["eps"])
    L = (Layer * cfg["layers"])()
    keep = []
    for i, lp in enumerate(params["layers"]):
        def a(v):
            v = np.ascontiguousarray(v)
            keep.append(v)
            return _p(v)
        L[i] = Layer(a(lp["attn_norm"]), a(lp["qkv"]["q4"]), a(lp["qkv"]["s"]), a(lp["qkv"]["b"]),
                     a(lp["q_norm"]), a(lp["k_norm"]), a(lp["o"]["q4"]), a(lp["o"]["s"]), a(lp["o"]["b"]),
                     a(lp["mlp_norm"]), a(lp["gate_up"]["q4"]), a(lp["gate_up"]["s"]), a(lp["gate_up"]["b"]),
                     a(lp["down"]["q4"]), a(lp["down"]["s"]), a(lp["down"]["b"]),
                     _p(cache["k"][i]), _p(cache["v"][i]))
    run_layers = cfg["layers"] if run_layers is None else run_layers
    run_vocab = cfg["vocab"] if run_vocab is None else run_vocab
    tok = np.ascontiguousarray(tokens, np.int32)
    B = tok.shape[0]
    logits = np.empty((B, run_vocab), np.float32)
    lib().oracle_decode_step(C.byref(c), L, _p(np.ascontiguousarray(params["embed"])),
                             _p(np.ascontiguousarray(params["norm"])), _p(np.ascontiguousarray(params["lm_head"])),
                             _p(tok), int(pos), B, _p(logits), run_layers, run_vocab)
    return logits
