"""Row reductions on the device against the oracle.  Shapes follow the
reference's softmax tests (tests/test_scan.py:35-48) and the benchmark configs."""
import ml_dtypes
import numpy as np
import pytest

from oracle import inputs, rownorm
from util import bf16, dev, host, pkg

pytestmark = pytest.mark.gpu


def _ulps(got, want, dtype, normwise=False):
    """≙ ulp_error of tests/metal_testing.py:99-117."""
    got = np.asarray(got).astype(np.float64)
    want = np.asarray(want).astype(np.float64)
    fin = np.isfinite(want)
    if not (np.array_equal(np.isnan(got), np.isnan(want)) and np.array_equal(got[~fin & ~np.isnan(want)], want[~fin & ~np.isnan(want)])):
        return np.inf
    if not fin.any():
        return 0.0
    fi = ml_dtypes.finfo(dtype)
    mag = np.abs(want[fin])
    if normwise:
        mag = np.full_like(mag, mag.max())
    ulp = np.exp2(np.floor(np.log2(np.maximum(mag, float(fi.smallest_normal)))) - fi.nmant)
    return float(np.max(np.abs(got[fin] - want[fin]) / ulp))


# the reference's own tolerances, tests/test_scan.py:90-93
ULPS = {("softmax", "float32"): 62, ("softmax", "float16"): 19, ("softmax", "bfloat16"): 1,
        ("log_softmax", "float32"): 2.1, ("log_softmax", "float16"): 2, ("log_softmax", "bfloat16"): 1}


@pytest.mark.parametrize("dtype,shape", [(np.float32, (33, 1000)), (np.float16, (33, 1000)), (bf16, (33, 1000)),
                                         (np.float32, (4, 16385))])
def test_softmax_reference_shapes(dtype, shape):
    p = pkg()
    x = (np.random.default_rng(0).standard_normal(shape) * 4).astype(dtype)
    name = np.dtype(dtype).name
    got = host(p.rows.softmax(dev(x)))
    assert _ulps(got, rownorm.softmax(x), dtype) <= ULPS[("softmax", name)]
    got = host(p.rows.log_softmax(dev(x)))
    assert _ulps(got, rownorm.log_softmax(x), dtype, normwise=True) <= ULPS[("log_softmax", name)]


def test_softmax_inf_nan_rows():
    p = pkg()
    x = np.random.default_rng(0).standard_normal((16, 256)).astype(np.float32)
    x[0, 3] = -np.inf
    x[1, :] = -np.inf
    x[2, 5] = np.nan
    got = host(p.rows.softmax(dev(x)))
    want = rownorm.softmax(x)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert got[0, 3] == 0.0
    np.testing.assert_allclose(got[~np.isnan(want)], want[~np.isnan(want)], rtol=1e-5, atol=1e-9)


def test_config4_rows():
    """bf16 RMSNorm over [M, 4096] and f32 softmax over [M*32, 2048] ~ N(0, 3)."""
    p = pkg()
    for m in (1, 8, 32):
        h, gain, logits = inputs.config4_rows(m)
        got = host(p.rows.rms_norm(dev(h), dev(gain), 1e-6))
        assert _ulps(got, rownorm.rms_norm(h, gain, 1e-6), bf16) <= 1
        got = host(p.rows.softmax(dev(logits)))
        np.testing.assert_allclose(got, rownorm.softmax(logits), rtol=1e-5, atol=1e-12)


def test_rms_norm_f32_rtol():
    p = pkg()
    x, w, b, gain = inputs.config1()
    got = host(p.rows.rms_norm(dev(x), dev(gain), 1e-6))
    np.testing.assert_allclose(got, rownorm.rms_norm(x, gain, 1e-6), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("shape", [(64, 1024), (8, 8192), (3, 70001), (5, 37), (2, 3)])
def test_layer_norm_and_long_rows(shape):
    p = pkg()
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(shape) * 0.5 + 1.0).astype(np.float32)
    got = host(p.rows.layer_norm(dev(x)))
    np.testing.assert_allclose(got, rownorm.layer_norm(x), rtol=2e-5, atol=2e-5)
    gain = (1 + 0.1 * rng.standard_normal(shape[-1])).astype(np.float32)
    beta = (0.1 * rng.standard_normal(shape[-1])).astype(np.float32)
    got = host(p.rows.layer_norm(dev(x), dev(gain), dev(beta)))
    np.testing.assert_allclose(got, rownorm.layer_norm(x, gain, beta), rtol=2e-5, atol=2e-5)
    got = host(p.rows.softmax(dev(x)))
    np.testing.assert_allclose(got, rownorm.softmax(x), rtol=2e-5, atol=1e-12)
    got = host(p.rows.rms_norm(dev(x), dev(gain), 1e-6))
    np.testing.assert_allclose(got, rownorm.rms_norm(x, gain, 1e-6), rtol=2e-5, atol=1e-7)


def test_in_place_and_empty():
    import torch
    p = pkg()
    x = np.random.default_rng(3).standard_normal((9, 515)).astype(np.float32)
    t = dev(x)
    p.rows.softmax(t, out=t)
    np.testing.assert_allclose(host(t), rownorm.softmax(x), rtol=1e-5, atol=1e-12)
    n0 = p.default_context().launch_count
    e = torch.empty((0, 128), device="cuda")
    assert p.rows.softmax(e).shape == (0, 128)
    assert p.default_context().launch_count == n0
    with pytest.raises(p.B200Error):
        p.rows.rownorm(7, t)
    with pytest.raises(p.B200Error):
        p.rows.rownorm(0, t)  # RMSNorm without a gain
