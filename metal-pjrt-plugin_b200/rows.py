"""Row reductions over the last dimension (RMSNorm, softmax, log_softmax,
LayerNorm): the jitted JAX forms of examples/llm/qwen3.py:294-297,325 and
bench/jax_bench.py:44-46, served by one kernel family."""
from . import _lib
from .context import default_context

KIND_RMS, KIND_SOFTMAX, KIND_LOG_SOFTMAX, KIND_LAYERNORM = 0, 1, 2, 3


def rownorm(kind, x, gain=None, beta=None, eps=1e-6, out=None, ctx=None, stream=None):
    import torch
    ctx = ctx or default_context(x.device.index or 0)
    assert x.is_contiguous()
    n = x.shape[-1] if x.dim() else 0
    rows = x.numel() // n if n else 0
    y = out if out is not None else torch.empty_like(x)
    _lib.check(_lib.lib().b200_rownorm(ctx.handle, stream or _lib.current_stream(), kind, _lib.ptr(x),
                                       _lib.ptr(gain), _lib.ptr(beta), _lib.ptr(y), rows, n,
                                       _lib.dtype_code(x.dtype), float(eps)))
    return y


def rms_norm(x, w, eps, **kw):
    return rownorm(KIND_RMS, x, gain=w, eps=eps, **kw)


def softmax(x, **kw):
    return rownorm(KIND_SOFTMAX, x, **kw)


def log_softmax(x, **kw):
    return rownorm(KIND_LOG_SOFTMAX, x, **kw)


def layer_norm(x, gain=None, beta=None, eps=1e-5, **kw):
    return rownorm(KIND_LAYERNORM, x, gain=gain, beta=beta, eps=eps, **kw)
