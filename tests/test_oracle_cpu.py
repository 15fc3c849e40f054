"""Self-consistency of the oracle: the benchmark quantisers round-trip, the C
restatement agrees with the NumPy one, seeded inputs are reproducible.  CPU only."""
import numpy as np

from oracle import cpu_ref, decoder, dense, inputs, quant, rownorm


def test_int4_pack_unpack_round_trip():
    rng = np.random.default_rng(0)
    q = rng.integers(0, 16, size=(7, 192)).astype(np.uint8)
    packed = quant.bl_pack_int4(q)
    assert packed.dtype == np.uint32 and packed.shape == (7, 24)
    assert np.array_equal(quant.bl_unpack_int4(packed), q)
    # little-endian along K: element 8i+j sits at bits 4j..4j+3
    assert (packed[0, 0] >> 4 * 3) & 0xF == q[0, 3]


def test_int4_quantiser_properties():
    x, packed, s, b, w = inputs.config4(1, 256, 64)
    q = quant.bl_unpack_int4(packed)
    assert q.min() >= 0 and q.max() <= 15
    wd = quant.dequant_f32(q, s, b)
    step = np.repeat(s.astype(np.float32), 64, axis=1)
    # reconstruction within one step (bf16 rounding of scale/offset included)
    assert np.all(np.abs(wd - w) <= step * 0.75 + 1e-3)
    # constant group: the 1e-12 guard keeps the scale finite
    w2 = np.zeros((2, 64), np.float32)
    p2, s2, b2 = quant.bl_quantize_int4(w2)
    assert np.isfinite(s2.astype(np.float32)).all() and np.all(quant.dequant_f32(quant.bl_unpack_int4(p2), s2, b2) == 0)


def test_int8_quantiser_properties():
    x, q, s, w = inputs.config3(1, 256, 32)
    assert s.shape == (32, 1) and q.dtype == np.int8 and np.abs(q).max() <= 127
    wd = quant.dequant_f32(q, s, None)
    # half a step, plus the bf16 rounding of the scale (up to 2^-8 relative) times |q| <= 127
    assert np.all(np.abs(wd - w) <= s.astype(np.float32) * 1.0 + 1e-6)
    qg, sg = quant.bl_quantize_int8(w, group=64)
    assert sg.shape == (32, 4)


def test_c_restatement_matches_numpy():
    x, packed, s, b, _ = inputs.config4(5, 512, 96)
    want = quant.qmm(x, quant.bl_unpack_int4(packed), s, b, np.float32)
    got = cpu_ref.qmv_int4(x, packed, s, b)
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-4 * np.sqrt(np.mean(want ** 2)) + 1e-5)
    x, q, s8, _ = inputs.config3(3, 512, 96)
    np.testing.assert_allclose(cpu_ref.qmv_int8(x, q, s8), quant.qmm(x, q, s8, None, np.float32), rtol=1e-4, atol=1e-4)
    xf, wf, bf, gain = inputs.config1(32, 128, 64)
    d = cpu_ref.gemm_f32(xf, wf, bf)
    want, _, _ = dense.gemm(xf, wf, bias=bf)
    np.testing.assert_allclose(d, want, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(cpu_ref.rms_norm_f32(d, gain, 1e-6), rownorm.rms_norm(d, gain, 1e-6), rtol=1e-5, atol=1e-6)
    lg = inputs.config4_rows(1, 64, 4, 128)[2]
    np.testing.assert_allclose(cpu_ref.softmax_f32(lg), rownorm.softmax(lg), rtol=1e-5, atol=1e-8)
    np.testing.assert_allclose(cpu_ref.layer_norm_f32(lg), rownorm.layer_norm(lg), rtol=1e-4, atol=1e-5)


def test_c_decoder_matches_numpy_decoder():
    cfg = inputs.decoder_config(layers=2, hidden=128, heads=4, kv_heads=2, head_dim=64, inter=256, vocab=512)
    params, cache, tokens = inputs.config5(cfg, batch=2, ctx=20, max_len=32)
    c1 = {k: [a.copy() for a in v] for k, v in cache.items()}
    c2 = {k: [a.copy() for a in v] for k, v in cache.items()}
    l1 = decoder.decode_step(params, tokens, c1, 20, cfg)
    l2 = cpu_ref.decode_step(params, tokens, c2, 20, cfg)
    # bf16 activations: two correct evaluations differ by rounding flips that
    # compound over layers; a flip at a 3-sigma logit alone is 0.023 x RMS
    assert dense.max_abs_over_rms(l2, l1) <= 6e-2
    assert np.array_equal(l1.argmax(-1), l2.argmax(-1))
    for li in range(2):
        assert np.abs(c1["k"][li].astype(np.float32) - c2["k"][li].astype(np.float32)).max() <= 0.07


def test_seeded_inputs_are_reproducible():
    a1 = inputs.config2(4, 64, 32)
    a2 = inputs.config2(4, 64, 32)
    for u, v in zip(a1, a2):
        assert np.array_equal(u.view(np.uint16), v.view(np.uint16))
    x, w, b, gain = inputs.config1(8, 16, 16)
    assert abs(float(w.std()) - 1 / 32) < 0.01 and abs(float(gain.mean()) - 1) < 0.2


def test_softmax_special_rows():
    x = np.random.default_rng(0).standard_normal((4, 16)).astype(np.float32)
    x[0, 3] = -np.inf
    x[1, :] = -np.inf
    x[2, 5] = np.nan
    y = rownorm.softmax(x)
    assert y[0, 3] == 0 and abs(y[0].sum() - 1) < 1e-6
    assert np.isnan(y[1]).all() and np.isnan(y[2]).all()
