"""Oracle: row reductions over the last dimension (test infrastructure).

RMSNorm follows examples/llm/qwen3.py:294-297, softmax / log_softmax the
max-subtract form jax.nn.softmax uses (call sites qwen3.py:325,
tests/test_scan.py:35-48), LayerNorm the benchmark form of
bench/jax_bench.py:44-46.  Statistics are accumulated in float64 ("true answer
for the rounded inputs", tests/metal_testing.py:6-13), the result is rounded
to f32 and then once to the input dtype.
"""
import numpy as np

KIND_RMS, KIND_SOFTMAX, KIND_LOG_SOFTMAX, KIND_LAYERNORM = 0, 1, 2, 3


def rms_norm(x, w, eps):
    x64 = np.asarray(x).astype(np.float64)
    y = x64 / np.sqrt(np.mean(x64 * x64, axis=-1, keepdims=True) + eps)
    return (y * np.asarray(w).astype(np.float64)).astype(np.float32).astype(np.asarray(x).dtype)


def softmax(x):
    """NaN anywhere in a row or a row of -inf gives a NaN row, like
    jax.nn.softmax (tests/test_scan.py:43-48)."""
    x64 = np.asarray(x).astype(np.float64)
    with np.errstate(invalid="ignore", over="ignore"):
        m = np.max(x64, axis=-1, keepdims=True)
        e = np.exp(x64 - m)
        y = e / np.sum(e, axis=-1, keepdims=True)
    return y.astype(np.float32).astype(np.asarray(x).dtype)


def log_softmax(x):
    x64 = np.asarray(x).astype(np.float64)
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        m = np.max(x64, axis=-1, keepdims=True)
        sh = x64 - m
        y = sh - np.log(np.sum(np.exp(sh), axis=-1, keepdims=True))
    return y.astype(np.float32).astype(np.asarray(x).dtype)


def layer_norm(x, gain=None, beta=None, eps=1e-5):
    x64 = np.asarray(x).astype(np.float64)
    mu = np.mean(x64, axis=-1, keepdims=True)
    var = np.mean((x64 - mu) ** 2, axis=-1, keepdims=True)
    y = (x64 - mu) / np.sqrt(var + eps)
    if gain is not None:
        y = y * np.asarray(gain).astype(np.float64)
    if beta is not None:
        y = y + np.asarray(beta).astype(np.float64)
    return y.astype(np.float32).astype(np.asarray(x).dtype)


def rownorm(kind, x, gain=None, beta=None, eps=1e-6):
    if kind == KIND_RMS:
        return rms_norm(x, gain if gain is not None else np.ones(x.shape[-1], np.float32), eps)
    if kind == KIND_SOFTMAX:
        return softmax(x)
    if kind == KIND_LOG_SOFTMAX:
        return log_softmax(x)
    if kind == KIND_LAYERNORM:
        return layer_norm(x, gain, beta, eps)
    raise ValueError(kind)
