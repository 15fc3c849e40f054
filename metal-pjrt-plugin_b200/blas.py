"""Dense GEMM with the fused epilogue, mirroring the reference's XLA-free
dispatch interface (metal_pjrt/blas/mps_gemm.h:23-53, steel_gemm.h:38-78):
GemmParams / MpsOperand / SteelEpilogue and run_steel_gemm(params, epilogue).
Tensors are torch CUDA tensors used as raw buffers."""
import ctypes as C
import dataclasses
from typing import Optional

from . import _lib
from .context import default_context

ACT_NONE, ACT_RELU, ACT_GELU, ACT_SILU = 0, 1, 2, 3


@dataclasses.dataclass
class Operand:
    """≙ MpsOperand: buffer, ld (elements between stored rows), batch_stride
    (0 = broadcast), transpose."""
    tensor: object
    ld: int
    batch_stride: int = 0
    transpose: bool = False

    def to_c(self):
        return _lib.Operand(self.tensor.data_ptr() if self.tensor is not None else None, self.ld,
                            self.batch_stride, _lib.dtype_code(self.tensor.dtype), int(self.transpose))


@dataclasses.dataclass
class GemmParams:
    """≙ GemmParams: C[b] (m x n) = alpha op(A[b]) op(B[b]) + beta C[b]."""
    m: int
    n: int
    k: int
    a: Operand
    b: Operand
    c: Operand
    batch_count: int = 1
    alpha: float = 1.0
    beta: float = 0.0

    def to_c(self):
        return _lib.GemmParamsC(self.m, self.n, self.k, self.batch_count, self.alpha, self.beta,
                                self.a.to_c(), self.b.to_c(), self.c.to_c())


@dataclasses.dataclass
class SteelEpilogue:
    """≙ SteelEpilogue: act 0 none / 1 ReLU / 2 GELU-tanh / 3 SiLU, bias (n
    elements of D's dtype), aux (D's layout, the pre-activation value)."""
    act: int = 0
    bias: Optional[object] = None
    aux: Optional[object] = None

    def to_c(self):
        return _lib.EpilogueC(self.act, self.bias.data_ptr() if self.bias is not None else None,
                              self.aux.data_ptr() if self.aux is not None else None)


def steel_gemm_supports(p: GemmParams, epi: Optional[SteelEpilogue] = None):
    """≙ SteelGemmSupports + the argument checks of RunSteelGemm. Returns (ok, why)."""
    pc = p.to_c()
    ec = (epi or SteelEpilogue()).to_c()
    st = _lib.lib().b200_gemm_validate(C.byref(pc), C.byref(ec))
    return st == _lib.OK, ("" if st == _lib.OK else _lib.lib().b200_last_error().decode())


def gemm_route(p: GemmParams, epi: Optional[SteelEpilogue] = None):
    """≙ ChooseGemv / ChooseSteelTile: which kernel would run."""
    pc = p.to_c()
    ec = (epi or SteelEpilogue()).to_c()
    return _lib.lib().b200_gemm_route(C.byref(pc), C.byref(ec))


def gemm_work(p: GemmParams):
    pc = p.to_c()
    return _lib.lib().b200_gemm_work(C.byref(pc))


def run_steel_gemm(p: GemmParams, epi: Optional[SteelEpilogue] = None, ctx=None, stream=None, route=0):
    """≙ RunSteelGemm / RunGemv: enqueue on the stream, return nothing, raise
    B200Error(INVALID_ARGUMENT / UNIMPLEMENTED / ...) like the absl::Status."""
    ctx = ctx or default_context(p.c.tensor.device.index or 0)
    pc = p.to_c()
    ec = (epi or SteelEpilogue()).to_c()
    L = _lib.lib()
    L.b200_gemm_force_route(ctx.handle, route)
    try:
        _lib.check(L.b200_gemm(ctx.handle, stream or _lib.current_stream(), C.byref(pc), C.byref(ec)))
    finally:
        L.b200_gemm_force_route(ctx.handle, 0)


def matmul(a, b, bias=None, act=ACT_NONE, out_dtype=None, transpose_b=False, ctx=None):
    """D = act(a @ op(b) + bias) for row-major 2-D tensors (the form XLA's
    GemmRewriter hands the reference as __cublas$lt$matmul)."""
    import torch
    m, k = a.shape
    n = b.shape[0] if transpose_b else b.shape[1]
    d = torch.empty((m, n), dtype=out_dtype or a.dtype, device=a.device)
    p = GemmParams(m, n, k, Operand(a, a.stride(0)), Operand(b, b.stride(0), transpose=transpose_b),
                   Operand(d, d.stride(0)))
    run_steel_gemm(p, SteelEpilogue(act, bias), ctx)
    return d
