"""The tcgen05 route of the int4 dequant-matmul (nibbles as e4m3 bytes in tensor memory, the
activations split into two e4m3 terms) against the oracle: the same cases and the same bound
as the streaming kernel, plus what is particular to it: tiles shared between CTAs, the exact
two-term split over a wide dynamic range, one-hot unpack order."""
import numpy as np
import pytest

from oracle import decoder as odec
from oracle import inputs, quant, rownorm
from util import bf16, dev, host, pkg, rel_rms_err

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture
def tc():
    p = pkg()
    ctx = p.default_context()
    p.lib().b200_qmm_force_route(ctx.handle, 2)
    yield p
    p.lib().b200_qmm_force_route(ctx.handle, 0)


def _w4(packed, s, b):
    return {"q4": dev(packed), "s": dev(s), "b": dev(b)}


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("k,n", [(256, 128), (1024, 520), (4096, 1024), (12288, 384)])
def test_product(tc, m, k, n):
    x, packed, s, b, _ = inputs.config4(m, k, n)
    want = quant.qmm(x, quant.bl_unpack_int4(packed), s, b, np.float32)
    got = host(tc.qwen3.linear(dev(x), _w4(packed, s, b))).astype(np.float32)
    assert rel_rms_err(got, want) <= TOL
    # the mma.sync kernel on the same inputs: both round the same f32 sums to bf16
    tc.lib().b200_qmm_force_route(tc.default_context().handle, 1)
    other = host(tc.qwen3.linear(dev(x), _w4(packed, s, b))).astype(np.float32)
    assert rel_rms_err(got, other) <= TOL
    assert tc.default_context().error() == 0


@pytest.mark.parametrize("m,k,n", [(1, 4096, 6144), (1, 4096, 24576), (8, 4096, 24576), (1, 12288, 4096), (4, 12288, 4096),
                                   (8, 12288, 4096)])
def test_qwen3_shapes(tc, m, k, n):
    """Full projection shapes (tiles shared by several CTAs); a sample of 512 columns is checked."""
    x, packed, s, b, _ = inputs.config4(m, k, n)
    wd = _w4(packed, s, b)
    got = host(tc.qwen3.linear(dev(x), wd)).astype(np.float32)
    again = host(tc.qwen3.linear(dev(x), wd)).astype(np.float32)
    assert np.array_equal(got, again)          # the shared tiles are summed in a fixed order
    cols = np.random.default_rng(0).choice(n, 512, replace=False)
    want = quant.qmm(x, quant.bl_unpack_int4(packed[cols]), s[cols], b[cols], np.float32)
    assert rel_rms_err(got[:, cols], want) <= TOL
    assert np.isfinite(got).all()


def test_one_hot_rows_return_the_dequantised_column(tc):
    k, n = 4096, 640
    _, packed, s, b, _ = inputs.config4(1, k, n)
    for ks in ([0, 1, 2, 3, 4, 5, 6, 7], [8, 15, 16, 31, 32, 33, 63, 64], [255, 256, 1000, 2047, 2048, 4032, 4094, 4095]):
        x = np.zeros((len(ks), k), np.float32)
        for i, kk in enumerate(ks):
            x[i, kk] = 1.0 if i % 2 == 0 else -3.0
        got = host(tc.qwen3.linear(dev(x.astype(bf16)), _w4(packed, s, b))).astype(np.float32)
        wd = quant.dequant_f32(quant.bl_unpack_int4(packed), s, b)
        want = wd[:, ks].T * x[np.arange(len(ks)), ks][:, None]
        ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(want), 1e-30))) - 7)
        assert np.all(np.abs(got - want) <= 0.51 * ulp + 1e-6)


def test_wide_dynamic_range_of_x(tc):
    """Elements of x from 2^-9 to 2^9 of the row's scale: the two-term e4m3 split holds every
    one within 2^10 of the largest exactly, and loses the rest below the bf16 rounding of the sum."""
    m, k, n = 2, 2048, 256
    _, packed, s, b, _ = inputs.config4(1, k, n)
    rng = np.random.default_rng(9)
    x = rng.standard_normal((m, k), dtype=np.float32) * np.exp2(rng.integers(-9, 10, size=(m, k))).astype(np.float32)
    x = x.astype(bf16)
    want = quant.qmm(x, quant.bl_unpack_int4(packed), s, b, np.float32)
    got = host(tc.qwen3.linear(dev(x), _w4(packed, s, b))).astype(np.float32)
    assert rel_rms_err(got, want) <= TOL


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("n", [512, 4096])
def test_fused_rmsnorm_prologue(tc, m, n):
    k = 1024
    x, packed, s, b, _ = inputs.config4(m, k, n)
    gain = (1 + 0.1 * np.random.default_rng(3).standard_normal(k, dtype=np.float32)).astype(bf16)
    h = rownorm.rms_norm(x, gain, 1e-6)
    want = quant.qmm(h, quant.bl_unpack_int4(packed), s, b, np.float32)
    got = host(tc.qwen3.linear(dev(x), _w4(packed, s, b), rms_gain=dev(gain), eps=1e-6)).astype(np.float32)
    assert rel_rms_err(got, want) <= TOL


@pytest.mark.parametrize("m", [1, 8])
def test_fused_silu_mul_prologue_and_residual(tc, m):
    k, n = 1536, 256
    _, packed, s, b, _ = inputs.config4(1, k, n)
    gu = (np.random.default_rng(8).standard_normal((m, 2 * k), dtype=np.float32) * 1.5).astype(bf16)
    act = odec.silu_mul(gu[:, :k], gu[:, k:])
    want = quant.qmm(act, quant.bl_unpack_int4(packed), s, b, np.float32)
    got = host(tc.qwen3.linear(dev(gu), _w4(packed, s, b), silu_mul=True)).astype(np.float32)
    assert got.shape == (m, n) and rel_rms_err(got, want) <= TOL
    res = np.random.default_rng(2).standard_normal((m, n), dtype=np.float32).astype(bf16)
    got_r = host(tc.qwen3.linear(dev(gu), _w4(packed, s, b), silu_mul=True, residual=dev(res))).astype(np.float32)
    want_r = (res.astype(np.float32) + want.astype(bf16).astype(np.float32)).astype(bf16).astype(np.float32)
    assert rel_rms_err(got_r, want_r) <= TOL


def test_zero_rows_of_x(tc):
    k, n = 512, 128
    _, packed, s, b, _ = inputs.config4(1, k, n)
    x = np.zeros((3, k), np.float32).astype(bf16)
    got = host(tc.qwen3.linear(dev(x), _w4(packed, s, b))).astype(np.float32)
    assert np.all(got == 0)
