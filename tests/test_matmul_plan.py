"""The BlasLt front of the dense GEMM: the twelve-epilogue table, the acceptance rules and
the row-major normal form on the CPU (≙ the rules of blas_lt_support.cc:25-201), and on the
device the reference's own parametrisation (metal_pjrt/blas/metal_blas_lt_test.cc:100-275):
12 epilogues x {f32, f16, bf16} x {row-, column-major output} x {5x7x3, 64x96x36}, batch 2,
with its data, its reference arithmetic and its tolerances."""
import ctypes as C

import numpy as np
import pytest

from util import bf16, dev, host, pkg

# (epilogue, bias, aux, act) as in kCases of the reference test
CASES = [(0, 0, 0, 0), (1, 0, 0, 1), (2, 1, 0, 0), (3, 1, 0, 1), (4, 0, 0, 2), (5, 0, 1, 2), (6, 1, 0, 2), (7, 1, 1, 2),
         (8, 0, 0, 3), (9, 0, 1, 3), (10, 1, 0, 3), (11, 1, 1, 3)]


def _layout(L, dtype, rows, cols, order, batch=1):
    ld = cols if order == L.ROW_MAJOR else rows
    return L.MatrixLayoutC(dtype, order, rows, cols, ld, batch, rows * cols, 0)


def _config(L, dtype, m, n, k, out_order, batch=1, out_dtype=None, beta=0.0):
    out = _layout(L, dtype if out_dtype is None else out_dtype, m, n, out_order, batch)
    return L.MatmulConfigC(_layout(L, dtype, m, k, L.ROW_MAJOR, batch), _layout(L, dtype, k, n, L.ROW_MAJOR, batch), out, out,
                           1.0, 0.0, beta)


def test_epilogue_table():
    p = pkg()
    L, lib = p._lib, p.lib()
    for code, bias, aux, act in CASES:
        spec = L.EpilogueSpecC()
        assert lib.b200_decode_epilogue(code, C.byref(spec)) == L.OK
        assert (spec.bias, spec.aux, spec.act) == (bias, aux, act)
    assert lib.b200_decode_epilogue(12, C.byref(L.EpilogueSpecC())) == L.UNIMPLEMENTED
    assert lib.b200_decode_epilogue(-1, C.byref(L.EpilogueSpecC())) == L.UNIMPLEMENTED


def test_normal_form_and_rules():
    p = pkg()
    L, lib = p._lib, p.lib()
    plan = L.MatmulPlanC()
    make = lambda cfg, epi=0: lib.b200_matmul_plan_create(C.byref(cfg), epi, C.byref(plan))
    # row-major output: as given
    assert make(_config(L, L.BF16, 5, 7, 3, L.ROW_MAJOR, batch=2), 10) == L.OK
    g = plan.params
    assert (plan.swap, g.m, g.n, g.k, g.batch) == (0, 5, 7, 3, 2)
    assert (g.a.ld, g.a.transpose, g.b.ld, g.b.transpose, g.c.ld, g.c.transpose) == (3, 0, 7, 0, 7, 0)
    assert (g.a.batch_stride, g.b.batch_stride, g.c.batch_stride) == (15, 21, 35)
    assert (plan.epi.bias, plan.epi.act, plan.epi.aux) == (1, 3, 0)
    # column-major output: D^T = B^T A^T, operands swapped, every layout seen transposed
    assert make(_config(L, L.BF16, 5, 7, 3, L.COLUMN_MAJOR, batch=2)) == L.OK
    g = plan.params
    assert (plan.swap, g.m, g.n, g.k) == (1, 7, 5, 3)
    assert (g.a.ld, g.a.transpose) == (7, 1)        # the old B (3 x 7 row-major) is now A^T's storage
    assert (g.b.ld, g.b.transpose) == (3, 1)        # the old A
    assert (g.c.ld, g.c.transpose) == (5, 0)        # the column-major 5 x 7 output is a row-major 7 x 5
    # an operand without a batch dimension is broadcast
    cfg = _config(L, L.F32, 4, 4, 4, L.ROW_MAJOR, batch=3)
    cfg.rhs.batch_size = 1
    assert make(cfg) == L.OK and plan.params.b.batch_stride == 0 and plan.params.a.batch_stride == 16
    cfg.out.batch_size = 2
    assert make(cfg) == L.INVALID_ARGUMENT          # output batch differs from the operands'
    # types: one operand type, result that type or f32
    cfg = _config(L, L.BF16, 4, 4, 4, L.ROW_MAJOR)
    cfg.rhs.dtype = L.F16
    assert make(cfg) == L.UNIMPLEMENTED and b"Cast the operands" in lib.b200_last_error()
    assert make(_config(L, L.BF16, 4, 4, 4, L.ROW_MAJOR, out_dtype=L.F32)) == L.OK
    assert make(_config(L, L.BF16, 4, 4, 4, L.ROW_MAJOR, out_dtype=L.F16)) == L.UNIMPLEMENTED
    # complex alpha, transpose flags, inconsistent shapes
    cfg = _config(L, L.F32, 4, 4, 4, L.ROW_MAJOR)
    cfg.alpha_imag = 1.0
    assert make(cfg) == L.UNIMPLEMENTED
    cfg = _config(L, L.F32, 4, 4, 4, L.ROW_MAJOR)
    cfg.lhs.transpose = 1
    assert make(cfg) == L.UNIMPLEMENTED
    cfg = _config(L, L.F32, 4, 5, 6, L.ROW_MAJOR)
    cfg.rhs.num_rows = 7
    assert make(cfg) == L.INVALID_ARGUMENT
    # beta != 0: C must be laid out exactly like D
    cfg = _config(L, L.F32, 4, 4, 4, L.ROW_MAJOR, beta=1.0)
    assert make(cfg) == L.OK
    cfg.c.leading_dim_stride = 8
    assert make(cfg) == L.UNIMPLEMENTED
    cfg.c.leading_dim_stride = 4
    cfg.c.order = L.COLUMN_MAJOR
    assert make(cfg) == L.UNIMPLEMENTED
    # 16-bit index limits (the reference's SteelOnlyShapeLimit): ld > INT32_MAX / 256 refused, f32 not limited
    k = (1 << 23) + 16
    for dt in (L.BF16, L.F16, L.F32):
        st = make(_config(L, dt, 2, 2, k, L.ROW_MAJOR))
        if dt == L.F32:
            assert st == L.OK
        else:
            assert st == L.UNIMPLEMENTED and b"leading dimension" in lib.b200_last_error()
    assert make(_config(L, L.F32, 4, 4, 4, L.ROW_MAJOR), 12) == L.UNIMPLEMENTED


def _round(a, dtype):
    if dtype == "f32":
        return a.astype(np.float32)
    return a.astype(np.float32).astype(np.float16 if dtype == "f16" else bf16).astype(np.float32)


def _act(act, x):
    if act == 1:
        return np.where(np.isnan(x), x, np.maximum(x, 0))
    if act == 2:
        return 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    if act == 3:
        return x / (1 + np.exp(-x))
    return x


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(5, 7, 3), (64, 96, 36)])
@pytest.mark.parametrize("order", ["row", "col"])
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_execute_with_every_epilogue(dtype, order, shape):
    import torch
    p = pkg()
    L, lib = p._lib, p.lib()
    ctx = p.default_context()
    m, n, k = shape
    batch = 2
    npdt = {"f32": np.float32, "f16": np.float16, "bf16": bf16}[dtype]
    code = {"f32": L.F32, "f16": L.F16, "bf16": L.BF16}[dtype]
    a = (((np.arange(batch * m * k) * 7) % 9) * 0.25 - 1.0).astype(np.float32).reshape(batch, m, k)
    b = (((np.arange(batch * k * n) * 5) % 11) * 0.25 - 1.25).astype(np.float32).reshape(batch, k, n)
    out_order = L.ROW_MAJOR if order == "row" else L.COLUMN_MAJOR
    bias_len = n if order == "row" else m          # along the output's minor dimension
    bias = (0.5 * np.arange(bias_len) - 1.0).astype(np.float32)
    ad, bd, biasd = dev(a.astype(npdt)), dev(b.astype(npdt)), dev(bias.astype(npdt))
    es = 4 if dtype == "f32" else 2
    tol = {"f32": 1e-5, "f16": 4e-3, "bf16": 2e-2}[dtype]
    acc = np.einsum("bik,bkj->bij", _round(a, dtype).astype(np.float64), _round(b, dtype).astype(np.float64))
    for epi, has_bias, has_aux, act in CASES:
        plan = L.MatmulPlanC()
        cfg = _config(L, code, m, n, k, out_order, batch)
        p._lib.check(lib.b200_matmul_plan_create(C.byref(cfg), epi, C.byref(plan)))
        d = torch.full((batch * m * n,), float("nan"), dtype=ad.dtype, device="cuda")
        aux = torch.full((batch * m * n,), float("nan"), dtype=ad.dtype, device="cuda")
        p._lib.check(lib.b200_matmul_execute(ctx.handle, p._lib.current_stream(), C.byref(plan), ad.data_ptr(), bd.data_ptr(),
                                             None, d.data_ptr(), biasd.data_ptr() if has_bias else None,
                                             aux.data_ptr() if has_aux else None, batch * m * n * es,
                                             bias_len * es if has_bias else 0, batch * m * n * es if has_aux else 0))
        torch.cuda.synchronize()
        pre = _round(acc, dtype).astype(np.float64)
        if has_bias:
            pre = pre + (_round(bias, dtype)[None, None, :] if order == "row" else _round(bias, dtype)[None, :, None])
        want = _act(act, pre)
        got = host(d).astype(np.float64).reshape((batch, m, n) if order == "row" else (batch, n, m))
        if order == "col":
            got = got.transpose(0, 2, 1)
        assert np.all(np.abs(got - want) <= tol * (1 + np.abs(want))), (epi, dtype, order)
        if has_aux:
            ga = host(aux).astype(np.float64).reshape((batch, m, n) if order == "row" else (batch, n, m))
            if order == "col":
                ga = ga.transpose(0, 2, 1)
            assert np.all(np.abs(ga - pre) <= tol * (1 + np.abs(pre))), (epi, dtype, order, "aux")
    assert ctx.error() == 0


@pytest.mark.gpu
def test_execute_seeds_d_with_c_and_checks_sizes():
    import torch
    p = pkg()
    L, lib = p._lib, p.lib()
    ctx = p.default_context()
    m, n, k = 8, 16, 32
    rng = np.random.default_rng(5)
    a, b, c = (rng.standard_normal(s, dtype=np.float32) for s in ((m, k), (k, n), (m, n)))
    ad, bd, cd = dev(a), dev(b), dev(c)
    d = torch.zeros((m, n), device="cuda")
    plan = L.MatmulPlanC()
    p._lib.check(lib.b200_matmul_plan_create(C.byref(_config(L, L.F32, m, n, k, L.ROW_MAJOR, beta=0.5)), 0, C.byref(plan)))
    p._lib.check(lib.b200_matmul_execute(ctx.handle, p._lib.current_stream(), C.byref(plan), ad.data_ptr(), bd.data_ptr(),
                                         cd.data_ptr(), d.data_ptr(), None, None, m * n * 4, 0, 0))
    torch.cuda.synchronize()
    assert np.allclose(host(d), a @ b + 0.5 * c, rtol=1e-5, atol=1e-5)
    assert np.array_equal(host(cd), c)                                  # C itself is untouched
    st = lib.b200_matmul_execute(ctx.handle, p._lib.current_stream(), C.byref(plan), ad.data_ptr(), bd.data_ptr(), cd.data_ptr(),
                                 d.data_ptr(), None, None, m * n * 4 - 1, 0, 0)
    assert st == L.INVALID_ARGUMENT                                     # D too small
    p._lib.check(lib.b200_matmul_plan_create(C.byref(_config(L, L.F32, m, n, k, L.ROW_MAJOR)), 2, C.byref(plan)))
    st = lib.b200_matmul_execute(ctx.handle, p._lib.current_stream(), C.byref(plan), ad.data_ptr(), bd.data_ptr(), None,
                                 d.data_ptr(), d.data_ptr(), None, m * n * 4, n * 4 - 4, 0)
    assert st == L.INVALID_ARGUMENT and b"bias" in lib.b200_last_error()
    assert ctx.error() == 0                                             # caller mistakes do not stick
