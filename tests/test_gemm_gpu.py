"""Dense GEMM with the fused epilogue against the float64 oracle, with the
reference's own tolerance formula and shape lists
(blas/steel_gemm_test.cc:174-211,227-344; blas/metal_blas_lt_test.cc:242-265),
canary padding around every output, and the benchmark's configs 1 and 2."""
import numpy as np
import pytest

from oracle import dense, inputs, rownorm
from util import bf16, dev, host, pkg

pytestmark = pytest.mark.gpu

NP = {"f32": np.float32, "f16": np.float16, "bf16": bf16}


def run_case(m, n, k, batch=1, dt_in="bf16", dt_out=None, ta=False, tb=False, alpha=1.0, beta=0.0, pad=0,
             broadcast_b=False, act=0, bias=False, aux=False, route=0, seed=0):
    import torch
    p = pkg()
    dt_out = dt_out or dt_in
    rng = np.random.default_rng(seed)
    ar, ac = (k, m) if ta else (m, k)
    br, bc = (n, k) if tb else (k, n)
    lda, ldb, ldd = ac + pad, bc + pad, n + pad
    A = rng.standard_normal((batch, ar, lda)).astype(NP[dt_in])
    B = rng.standard_normal((1 if broadcast_b else batch, br, ldb)).astype(NP[dt_in])
    D0 = rng.standard_normal((batch, m, ldd)).astype(NP[dt_out])
    bias_h = rng.standard_normal((n,)).astype(NP[dt_out]) if bias else None
    At, Bt, Dt = dev(A), dev(B), dev(D0)
    aux_t = torch.full_like(Dt, 7.0) if aux else None
    bias_t = dev(bias_h) if bias else None
    B_ = p.blas
    prm = B_.GemmParams(m, n, k, B_.Operand(At, lda, ar * lda, ta),
                        B_.Operand(Bt, ldb, 0 if broadcast_b else br * ldb, tb),
                        B_.Operand(Dt, ldd, m * ldd), batch, alpha, beta)
    B_.run_steel_gemm(prm, B_.SteelEpilogue(act, bias_t, aux_t), route=route)
    got = host(Dt).astype(np.float64)
    a_log = A[:, :, :ac]
    b_log = np.broadcast_to(B[:, :, :bc], (batch, br, bc))
    want, want_aux, mag = dense.gemm(a_log, b_log, ta=ta, tb=tb, alpha=alpha, beta=beta, c=D0[:, :, :n],
                                     bias=bias_h, activation=act, out_dtype=NP[dt_out], want_aux=aux)
    # tolerance on the pre-activation magnitude (steel_gemm_test.cc:195-196); activations are 1-Lipschitz-ish
    v = alpha * (np.swapaxes(a_log, -1, -2) if ta else a_log).astype(np.float64) @ \
        (np.swapaxes(b_log, -1, -2) if tb else b_log).astype(np.float64)
    if beta != 0:
        v = v + beta * D0[:, :, :n].astype(np.float64)
    if bias:
        v = v + bias_h.astype(np.float64)
    want64 = dense.act(act, v)
    tol = dense.tolerance(want64, mag + (np.abs(bias_h.astype(np.float64)) if bias else 0), k, NP[dt_out]) * 1.13
    err = np.abs(got[:, :, :n] - want64)
    assert np.all(err <= tol), f"max err {err.max()} (tol {tol.flat[np.argmax(err)]})"
    # padding between rows must be untouched (steel_gemm_test.cc:203-211)
    if pad:
        assert np.array_equal(host(Dt)[:, :, n:].view(np.uint8), D0[:, :, n:].view(np.uint8))
    if aux:
        ga = host(aux_t).astype(np.float64)
        tol_aux = dense.tolerance(v, mag + (np.abs(bias_h.astype(np.float64)) if bias else 0), k, NP[dt_out]) * 1.13
        assert np.all(np.abs(ga[:, :, :n] - v) <= tol_aux)
        if pad:
            assert np.all(ga[:, :, n:] == 7.0)


SHAPES = [(1, 1, 1), (3, 5, 7), (16, 16, 16), (64, 64, 64), (65, 63, 17), (128, 96, 40), (257, 31, 33),
          (48, 200, 130), (5, 7, 3), (64, 96, 36)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_transposes_and_unaligned(m, n, k, ta, tb):
    run_case(m, n, k, ta=ta, tb=tb, pad=3)


@pytest.mark.parametrize("dt_in,dt_out", [("f32", "f32"), ("f16", "f16"), ("bf16", "bf16"), ("f16", "f32"), ("bf16", "f32")])
def test_dtype_combinations(dt_in, dt_out):
    run_case(70, 50, 90, dt_in=dt_in, dt_out=dt_out, pad=2)
    run_case(33, 65, 4096, dt_in=dt_in, dt_out=dt_out)   # long K (steel_gemm_test.cc K=4096)


def test_alpha_beta_batched_broadcast_k0():
    run_case(40, 24, 56, alpha=0.5, beta=0.0)
    run_case(40, 24, 56, alpha=-1.5, beta=0.75, pad=1)
    run_case(40, 24, 56, batch=3, beta=1.0)
    run_case(40, 24, 56, batch=3, broadcast_b=True, tb=True)
    run_case(9, 11, 0, beta=0.5)      # K = 0: D = beta * D
    run_case(9, 11, 0, beta=0.0, bias=True, act=1)


@pytest.mark.parametrize("act", [0, 1, 2, 3])
@pytest.mark.parametrize("bias,aux", [(False, False), (True, False), (True, True), (False, True)])
@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
def test_epilogues(act, bias, aux, dt):
    """The 12 BlasLt epilogues x dtypes (blas/metal_blas_lt_test.cc:242-265)."""
    run_case(64, 96, 36, dt_in=dt, act=act, bias=bias, aux=aux, pad=4, batch=2)
    run_case(5, 7, 3, dt_in=dt, act=act, bias=bias, aux=aux)


def test_relu_keeps_nan():
    import torch
    p = pkg()
    a = torch.full((4, 8), float("nan"), device="cuda")
    b = torch.ones((8, 4), device="cuda")
    d = p.blas.matmul(a, b, act=1)
    assert torch.isnan(d).all()


@pytest.mark.parametrize("vecs", [1, 2, 3, 5, 8, 17, 32])
@pytest.mark.parametrize("vectors_are_b", [False, True])
def test_few_row_route(vecs, vectors_are_b):
    """x . W^T with few rows on either side (≙ gemv_test.cc:246-312, every vector
    count, both orientations, with epilogues)."""
    p = pkg()
    m, n = (516 + 12, vecs) if vectors_are_b else (vecs, 516 + 12)
    for k in (1024, 576):
        run_case(m, n, k, tb=True, route=p._lib.ROUTE_FEWROW, bias=True, act=3, aux=True, seed=vecs)
    B_ = p.blas
    A, Bm, D = dev(np.zeros((m, 1024), bf16)), dev(np.zeros((n, 1024), bf16)), dev(np.zeros((m, n), bf16))
    prm = B_.GemmParams(m, n, 1024, B_.Operand(A, 1024), B_.Operand(Bm, 1024, transpose=True), B_.Operand(D, n))
    # up to 8 vectors the streaming kernel is the library's choice, above that the tensor-core route
    assert B_.gemm_route(prm) == (p._lib.ROUTE_FEWROW if vecs <= 8 else p._lib.ROUTE_TCGEN05)


def test_config1_f32_block():
    """x[512,1024] @ W[1024,1024] + b, then RMSNorm: f32, rtol 1e-5."""
    p = pkg()
    x, w, b, gain = inputs.config1()
    d = p.blas.matmul(dev(x), dev(w), bias=dev(b))
    y = host(p.rows.rms_norm(d, dev(gain), 1e-6))
    lin, _, _ = dense.gemm(x, w, bias=b)
    # reference in float64 end to end
    v = x.astype(np.float64) @ w.astype(np.float64) + b.astype(np.float64)
    want = v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + 1e-6) * gain.astype(np.float64)
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(host(d), lin, rtol=1e-5, atol=2e-5)


@pytest.mark.parametrize("m", [1, 16, 128])
def test_config2_bias_silu(m):
    """bf16 A[M,4096] @ B[4096,4096] + bias, SiLU, f32 accumulate: max-abs <= 2e-2 x RMS."""
    p = pkg()
    a, b, bias = inputs.config2(m)
    d = host(p.blas.matmul(dev(a), dev(b), bias=dev(bias), act=3)).astype(np.float64)
    v = a.astype(np.float64) @ b.astype(np.float64) + bias.astype(np.float64)
    want = dense.act(3, v)
    assert dense.max_abs_over_rms(d, want) <= 2e-2


# ---- the tensor-core (tcgen05) route -------------------------------------------------------

def _tc_case(m, n, k, ta=False, tb=False, dt_in="bf16", dt_out=None, alpha=1.0, beta=0.0, act=0, bias=False,
             aux=False, seed=0):
    """Like run_case but with 16-byte-aligned leading dimensions, asserting the route."""
    import torch
    p = pkg()
    dt_out = dt_out or dt_in
    rng = np.random.default_rng(seed)
    r8 = lambda v: (v + 7) // 8 * 8
    ar, ac = (k, m) if ta else (m, k)
    br, bc = (n, k) if tb else (k, n)
    lda, ldb, ldd = r8(ac), r8(bc), r8(n) + 8
    A = rng.standard_normal((ar, lda)).astype(NP[dt_in])
    B = (rng.standard_normal((br, ldb)) * 0.5).astype(NP[dt_in])
    D0 = rng.standard_normal((m, ldd)).astype(NP[dt_out])
    bias_h = rng.standard_normal((n,)).astype(NP[dt_out]) if bias else None
    At, Bt, Dt = dev(A), dev(B), dev(D0)
    aux_t = torch.full_like(Dt, 7.0) if aux else None
    bias_t = dev(bias_h) if bias else None
    B_ = p.blas
    prm = B_.GemmParams(m, n, k, B_.Operand(At, lda, 0, ta), B_.Operand(Bt, ldb, 0, tb), B_.Operand(Dt, ldd), 1, alpha, beta)
    epi = B_.SteelEpilogue(act, bias_t, aux_t)
    # few-row x . W^T shapes prefer the streaming kernel; force the tensor-core route here
    assert B_.gemm_route(prm, epi) in (p._lib.ROUTE_TCGEN05, p._lib.ROUTE_FEWROW)
    B_.run_steel_gemm(prm, epi, route=p._lib.ROUTE_TCGEN05)
    torch.cuda.synchronize()
    assert p.default_context().error() == 0
    a_log, b_log = A[:, :ac].astype(np.float64), B[:, :bc].astype(np.float64)
    if ta:
        a_log = a_log.T
    if tb:
        b_log = b_log.T
    v = alpha * (a_log @ b_log)
    mag = abs(alpha) * (np.abs(a_log) @ np.abs(b_log))
    if beta != 0:
        v = v + beta * D0[:, :n].astype(np.float64)
        mag = mag + np.abs(beta * D0[:, :n].astype(np.float64))
    if bias:
        v = v + bias_h.astype(np.float64)
        mag = mag + np.abs(bias_h.astype(np.float64))
    want = dense.act(act, v)
    got = host(Dt).astype(np.float64)
    tol = dense.tolerance(want, mag, k, NP[dt_out]) * 1.13
    err = np.abs(got[:, :n] - want)
    assert np.all(err <= tol), f"max err {err.max()} at {np.unravel_index(np.argmax(err - tol), err.shape)}"
    assert np.array_equal(host(Dt)[:, n:].view(np.uint8), D0[:, n:].view(np.uint8))   # padding untouched
    if aux:
        ga = host(aux_t).astype(np.float64)
        assert np.all(np.abs(ga[:, :n] - v) <= dense.tolerance(v, mag, k, NP[dt_out]) * 1.13)
        assert np.all(ga[:, n:] == 7.0)


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 128, 128), (256, 512, 320), (200, 264, 136), (33, 40, 72),
                                   (1, 4096, 512), (300, 1000, 1024)])
def test_tcgen05_layouts_and_ragged_edges(m, n, k, ta, tb):
    _tc_case(m, n, k, ta=ta, tb=tb, seed=m + n)


@pytest.mark.parametrize("dt_in,dt_out", [("bf16", "bf16"), ("f16", "f16"), ("bf16", "f32"), ("f16", "f32")])
def test_tcgen05_dtypes_and_epilogues(dt_in, dt_out):
    for act in (0, 1, 2, 3):
        _tc_case(160, 288, 192, dt_in=dt_in, dt_out=dt_out, act=act, bias=True, aux=(act % 2 == 1), seed=act)
    _tc_case(160, 288, 192, dt_in=dt_in, dt_out=dt_out, alpha=-0.5, beta=0.75)


@pytest.mark.parametrize("dt_in,dt_out", [("bf16", "bf16"), ("f16", "f32")])
def test_tcgen05_split_k_cluster(dt_in, dt_out):
    """Few tiles and a long K: the K loop is split across a cluster of CTAs whose partial
    tiles are added through distributed shared memory; every epilogue part, ragged K."""
    for m, n, k in ((100, 200, 1000), (16, 520, 2048), (128, 1024, 4096), (7, 136, 8200)):
        _tc_case(m, n, k, dt_in=dt_in, dt_out=dt_out, act=3, bias=True, aux=True, seed=k)
        _tc_case(m, n, k, dt_in=dt_in, dt_out=dt_out, tb=True, alpha=-0.5, beta=0.75, seed=k + 1)
    _tc_case(100, 200, 1000, dt_in=dt_in, dt_out=dt_out, ta=True, tb=True, act=1, seed=5)


def test_tcgen05_many_tiles_persistent():
    """More tiles than SMs, so every CTA walks several tiles and both accumulators rotate."""
    _tc_case(2048, 2560, 256, bias=True, act=3)
    _tc_case(1536, 4096, 512, tb=True)


@pytest.mark.parametrize("m", [2048, 8192])
def test_config2_large_m_properties(m):
    """Config 2 at the sizes the CPU cannot check in full: a sample of rows against the
    float64 oracle, and linearity in A (rows scaled by powers of two scale exactly)."""
    import torch
    p = pkg()
    a, b, bias = inputs.config2(m)
    ad, bd, biasd = dev(a), dev(b), dev(bias)
    d = p.blas.matmul(ad, bd, bias=biasd, act=3)
    rows = np.random.default_rng(0).choice(m, 24, replace=False)
    v = a[rows].astype(np.float64) @ b.astype(np.float64) + bias.astype(np.float64)
    assert dense.max_abs_over_rms(host(d)[rows].astype(np.float64), dense.act(3, v)) <= 2e-2
    lin1 = p.blas.matmul(ad, bd)
    lin2 = p.blas.matmul(ad * 2, bd)
    assert torch.equal(lin2, lin1 * 2)
