"""B200-native hot path of the jax-graft plugin, behind its operator surface.

The product is libb200graft.so (hand-written sm_100a CUDA behind the C ABI of
include/b200graft.h).  This package is the thin host side: `_lib` binds the C
ABI with ctypes, `blas` mirrors the reference's GemmParams / SteelEpilogue /
RunSteelGemm dispatch interface (metal_pjrt/blas/steel_gemm.h), `qwen3` mirrors
the model-level functions of examples/llm/qwen3.py (quantised `linear`,
`rms_norm`, the decode step).  torch is used only as a holder of device memory
and streams; no computation happens in Python and nothing falls back to the CPU.
"""
from . import _lib
from ._lib import B200Error, lib
from .context import Context, default_context
from . import blas, loader, qwen3, rows

__all__ = ["_lib", "B200Error", "lib", "Context", "default_context", "blas", "loader", "qwen3", "rows"]
