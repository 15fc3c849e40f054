"""The C-ABI library loads, exports every symbol include/b200graft.h declares,
and its pure (no-device) entry points behave.  CPU only."""
import ctypes as C
import os
import re

import pytest

from util import ROOT, pkg


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200graft.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    p = pkg()
    lib = p.lib()
    names = _declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
        assert n in p._lib.PROTOTYPES, f"{n} has no ctypes prototype"
    assert sorted(p._lib.PROTOTYPES) == names
    assert lib.b200_abi_version() == 1


def test_header_compiles_as_c():
    import subprocess
    src = '#include "b200graft.h"\nint main(void){return B200_ABI_VERSION-1;}\n'
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-x", "c", "-",
                        "-fsyntax-only"], input=src, text=True, capture_output=True)
    assert r.returncode == 0, r.stderr


def _gemm(p, m, n, k, dtype=2, out_dtype=None, ta=0, tb=0, lda=None, ldb=None, ldc=None, batch=1, beta=0.0,
          ptr=4096):
    L = p._lib
    a = L.Operand(ptr, lda if lda is not None else (m if ta else k), 0, dtype, ta)
    b = L.Operand(ptr, ldb if ldb is not None else (k if tb else n), 0, dtype, tb)
    c = L.Operand(ptr, ldc if ldc is not None else n, 0, dtype if out_dtype is None else out_dtype, 0)
    return L.GemmParamsC(m, n, k, batch, 1.0, beta, a, b, c)


def test_gemm_validate_rules():
    """The acceptance rules of SteelGemmSupports / RunSteelGemm
    (metal_pjrt/blas/steel_gemm.cc:140-196), checked without a device."""
    p = pkg()
    L, lib = p._lib, p.lib()
    epi = L.EpilogueC(0, None, None)
    ok = lambda g, e=epi: lib.b200_gemm_validate(C.byref(g), C.byref(e))
    assert ok(_gemm(p, 64, 64, 64)) == L.OK
    assert ok(_gemm(p, 1, 1, 1)) == L.OK
    assert ok(_gemm(p, 0, 5, 7, ptr=None)) == L.OK                      # empty problems are fine
    assert ok(_gemm(p, 5, 7, 0)) == L.OK                                # K = 0: D = beta * D
    g = _gemm(p, 8, 8, 8); g.b.dtype = L.F16
    assert ok(g) == L.INVALID_ARGUMENT                                   # A and B dtypes differ
    assert ok(_gemm(p, 8, 8, 8, dtype=L.BF16, out_dtype=L.F16)) == L.INVALID_ARGUMENT
    assert ok(_gemm(p, 8, 8, 8, dtype=L.BF16, out_dtype=L.F32)) == L.OK  # f32 output is allowed
    g = _gemm(p, 8, 8, 8); g.c.transpose = 1
    assert ok(g) == L.INVALID_ARGUMENT                                   # transposed C
    assert ok(_gemm(p, -1, 8, 8)) == L.INVALID_ARGUMENT
    assert ok(_gemm(p, 8, 8, 8, lda=7)) == L.INVALID_ARGUMENT            # ld < row length
    assert ok(_gemm(p, 8, 8, 8, ldc=7)) == L.INVALID_ARGUMENT
    assert ok(_gemm(p, 8, 8, 8, lda=(2**31 - 1) // 256 + 1)) == L.INVALID_ARGUMENT   # ld limit 8388607
    assert ok(_gemm(p, 8, 8, 8, lda=(2**31 - 1) // 256)) == L.OK
    assert ok(_gemm(p, 8, 8, 8, ptr=None)) == L.INVALID_ARGUMENT         # null buffer
    assert ok(_gemm(p, 8, 8, 8), L.EpilogueC(4, None, None)) == L.INVALID_ARGUMENT  # unknown activation
    assert b"activation" in lib.b200_last_error()
    g = _gemm(p, 8, 8, 8); g.a.batch_stride = -1
    assert ok(g) == L.INVALID_ARGUMENT


def test_gemm_route_table():
    """≙ the plan table of blas/gemv_test.cc:314-379: which shapes take the
    few-row streaming kernel."""
    p = pkg()
    L, lib = p._lib, p.lib()
    epi = L.EpilogueC(0, None, None)
    route = lambda g: lib.b200_gemm_route(C.byref(g), C.byref(epi))
    assert route(_gemm(p, 0, 8, 8)) == L.ROUTE_NONE
    for m in (1, 2, 5, 8, 32):
        assert route(_gemm(p, m, 4096, 1024, tb=1)) == L.ROUTE_FEWROW                # x . W^T, few rows of x
        assert route(_gemm(p, 4096, m, 1024, tb=1)) == L.ROUTE_FEWROW                # few rows on the other side
    assert route(_gemm(p, 33, 4096, 1024, tb=1)) != L.ROUTE_FEWROW
    assert route(_gemm(p, 4, 4096, 448, tb=1)) != L.ROUTE_FEWROW                     # K below 512
    assert route(_gemm(p, 4, 4096, 1000, tb=1)) != L.ROUTE_FEWROW                    # K not a multiple of 64
    assert route(_gemm(p, 4, 4096, 1024, tb=0)) != L.ROUTE_FEWROW                    # NN layout
    assert route(_gemm(p, 4, 4096, 1024, tb=1, dtype=L.F16)) != L.ROUTE_FEWROW
    assert route(_gemm(p, 4, 4096, 1024, tb=1, beta=1.0)) != L.ROUTE_FEWROW
    assert route(_gemm(p, 4, 4096, 1024, tb=1, batch=2)) != L.ROUTE_FEWROW
    assert route(_gemm(p, 4, 4096, 1024, tb=1, ldb=1032)) != L.ROUTE_FEWROW          # padded matrix rows
    assert route(_gemm(p, 512, 1024, 1024, dtype=L.F32)) == L.ROUTE_SIMT             # true f32 stays SIMT


def test_gemm_work():
    p = pkg()
    g = _gemm(p, 128, 4096, 4096)
    assert p.lib().b200_gemm_work(C.byref(g)) == 2 * 128 * 4096 * 4096
    g = _gemm(p, 1, 4096, 4096)
    assert p.lib().b200_gemm_work(C.byref(g)) == 64 * 2 * (4096 + 4096 * 4096 + 4096)


def test_qmm_validate_and_plan():
    p = pkg()
    L, lib = p._lib, p.lib()

    def q(bits=4, group=64, M=1, N=4096, K=4096, order=0, ptr=4096, epi=0):
        s = L.QmmParamsC()
        s.bits, s.group, s.nibble_order, s.epilogue, s.M, s.N, s.K = bits, group, order, epi, M, N, K
        s.x = s.q = s.scale = s.bias = s.out = ptr
        return s
    v = lambda s: lib.b200_qmm_validate(C.byref(s))
    assert v(q()) == L.OK
    assert v(q(bits=5)) == L.INVALID_ARGUMENT
    assert v(q(M=33)) == L.OK                       # beyond the streaming kernel: panel-wise dequantise + GEMM
    assert v(q(M=33, epi=2)) == L.UNIMPLEMENTED     # ... which has no "bf16-rounded value in f32" output
    s33 = q(M=33)
    s33.prologue = 2
    assert v(s33) == L.UNIMPLEMENTED                # ... and fuses no input transform
    assert v(q(K=4000)) == L.UNIMPLEMENTED
    assert v(q(group=32)) == L.UNIMPLEMENTED
    assert v(q(bits=8, group=4096)) == L.OK         # per output channel
    assert v(q(bits=8, group=128)) == L.UNIMPLEMENTED
    assert v(q(order=2)) == L.INVALID_ARGUMENT
    assert v(q(M=0, ptr=None)) == L.OK
    assert v(q(ptr=None)) == L.INVALID_ARGUMENT
    assert v(q(ptr=4100)) == L.INVALID_ARGUMENT     # packed weights must be 16-byte aligned
    assert v(q(epi=1)) == L.INVALID_ARGUMENT        # residual epilogue without a residual
    assert v(q(epi=4, N=24576)) == L.OK             # silu(gate) * up in the epilogue of a row-interleaved gate_up
    assert v(q(epi=4, N=24584)) == L.UNIMPLEMENTED  # ... whose rows come in sixteens
    assert v(q(epi=4, M=9)) == L.UNIMPLEMENTED      # ... for up to 8 rows of x
    assert v(q(epi=4, bits=16)) == L.UNIMPLEMENTED
    assert v(q(epi=5)) == L.INVALID_ARGUMENT
    # plans: tiles grow with the batch block count; small matrices split K across a cluster
    plan = p.qwen3.qmm_plan
    assert plan(1, 4096, 4096) == (32, 1, 1)       # one 32-row tile for 128 CTAs costs the busiest SM what two 16-row tiles would
    assert plan(1, 6144, 4096) == (32, 1, 1) and plan(1, 2048, 4096)[0] == 16
    assert plan(1, 1024, 4096)[1] == 1              # 64 CTAs without a K split beat 64 clusters of four (measured)
    assert plan(1, 256, 4096)[1] >= 2               # a handful of tiles: K is split across a cluster
    assert plan(8, 4096, 4096) == (16, 1, 1)        # persistent CTAs stage x once: no need for taller tiles
    assert plan(16, 4096, 4096)[0] == 32 and plan(16, 4096, 4096)[2] == 2
    r32, s32, mb32 = plan(32, 4096, 12288)
    assert mb32 == 4 and 32 * (12288 // s32) * 2 <= 96 * 1024
    # every batch size up to 32 has a plan for the decoder's projection shapes, in all three formats
    for n, k in ((6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288), (151936, 4096)):
        for m in range(1, 33):
            for bits, group in ((4, 64), (8, 64), (8, k), (16, 0)):
                assert plan(m, n, k, bits=bits, group=group)[0] in (16, 32, 64)


def test_no_device_means_a_loud_failure():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    p = pkg()
    with pytest.raises(p.B200Error) as e:
        p.Context(0)
    assert e.value.status == p._lib.FAILED_PRECONDITION and "no CPU fallback" in str(e.value)


def test_peer_exchange_rejects_bad_arguments():
    """The peer-exchange entry points validate before touching a device."""
    p = pkg()
    L, lib = p._lib, p.lib()
    buf = (C.c_char * L.TP_PEER_HANDLE_BYTES)()
    assert lib.b200_tp_peer_alloc(None, 1024, buf) == L.INVALID_ARGUMENT
    assert lib.b200_tp_peer_connect(None, buf) == L.INVALID_ARGUMENT
    assert not lib.b200_tp_peer_partial(None, 0)
    assert lib.b200_tp_sum_residual_norm(None, None, 0, None, None, None, 1, 64, 1e-6) == L.FAILED_PRECONDITION
