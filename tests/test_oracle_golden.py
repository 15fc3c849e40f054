"""The oracle against the fixtures generated from the reference's own code
(tests/golden/make_golden.py).  CPU only."""
import os

import ml_dtypes
import numpy as np

from oracle import decoder, quant, rownorm

bf16 = ml_dtypes.bfloat16


def _bf(a):
    return np.asarray(a).view(bf16)


def _ulps_bf16(got, want):
    g = np.asarray(got).astype(np.float64)
    w = np.asarray(want).astype(np.float64)
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(w), 1e-30))) - 7)
    return float(np.max(np.abs(g - w) / ulp))


def test_reference_quantisers_bit_exact(golden_dir):
    z = np.load(os.path.join(golden_dir, "quant_ref.npz"))
    q8, s8 = quant.ref_quantize_int8(z["w"])
    assert np.array_equal(q8, z["q8"]) and np.array_equal(s8, z["s8"])
    p4, s4, b4 = quant.ref_quantize_int4(z["w"])
    assert np.array_equal(p4, z["p4"])
    assert np.array_equal(s4, z["s4"]) and np.array_equal(b4, z["b4"])


def test_reference_dequantize_bit_exact(golden_dir):
    z = np.load(os.path.join(golden_dir, "quant_ref.npz"))
    d4 = quant.ref_dequantize_int4(z["p4"], z["s4"], z["b4"])
    assert np.array_equal(d4.view(np.uint16), z["deq4"])
    d8 = quant.ref_dequantize_int8(z["q8"], z["s8"])
    assert np.array_equal(d8.view(np.uint16), z["deq8"])


def test_reference_matvec(golden_dir):
    z = np.load(os.path.join(golden_dir, "quant_ref.npz"))
    x = _bf(z["x"])
    mv8 = quant.ref_matvec_int8(x, z["q8"], z["s8"].astype(bf16))
    mv4 = quant.ref_matvec_int4(x, z["p4"], z["s4"].astype(bf16), z["b4"].astype(bf16))
    # the fixture sums in f32 (NumPy pairwise), the oracle in f64: one bf16 ulp
    assert _ulps_bf16(mv8, _bf(z["mv8"])) <= 1.0
    assert _ulps_bf16(mv4, _bf(z["mv4"])) <= 1.0


def test_split_half_and_sequential_layouts_agree(golden_dir):
    z = np.load(os.path.join(golden_dir, "quant_ref.npz"))
    seq = quant.split_half_to_seq(z["p4"])
    q_ref = quant.ref_unpack_int4(z["p4"]).reshape(z["p4"].shape[0], -1)
    assert np.array_equal(quant.bl_unpack_int4(seq), q_ref)
    # same product through the generic oracle path (f32 dequant, f64 sum)
    x = _bf(z["x"])
    G = z["p4"].shape[1]
    y = quant.qmm(x, q_ref, z["s4"].astype(bf16).reshape(-1, G), z["b4"].astype(bf16).reshape(-1, G))
    assert _ulps_bf16(y, _bf(z["mv4"])) <= 1.0


def test_rows_against_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "rows_ref.npz"))
    y = rownorm.rms_norm(_bf(z["xr"]), _bf(z["gain"]), 1e-6)
    assert _ulps_bf16(y, _bf(z["rms_bf16"])) <= 1.0
    y32 = rownorm.rms_norm(z["xr32"], z["gain32"], 1e-6)
    np.testing.assert_allclose(y32, z["rms_f32"], rtol=1e-5, atol=1e-7)
    xh = _bf(z["xh"])                                      # [B, 1, H, D]
    r = decoder.rope(xh[:, 0], np.array([7, 7]), 1e6)
    assert _ulps_bf16(r, _bf(z["rope"])[:, 0]) <= 1.0
    q = _bf(z["q"])[:, 0]
    a = decoder.attention_decode(q, _bf(z["kc"]), _bf(z["vc"]), 18, 64 ** -0.5)
    assert _ulps_bf16(a, _bf(z["attn"])[:, 0]) <= 1.0


def test_decoder_forward_against_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "decoder_ref.npz"))
    cfg = dict(layers=2, hidden=128, heads=4, kv_heads=2, head_dim=64, inter=256,
               vocab=320, theta=1e6, eps=1e-6)
    layers = []
    for li in range(2):
        lp = {}
        for name in ("attn_norm", "q_norm", "k_norm", "mlp_norm"):
            lp[name] = _bf(z[f"l{li}_{name}"])
        for name in ("qkv", "o", "gate_up", "down"):
            lp[name] = {"q4h": z[f"l{li}_{name}_q4"], "s": _bf(z[f"l{li}_{name}_s"]),
                        "b": _bf(z[f"l{li}_{name}_b"])}
        layers.append(lp)
    params = {"embed": _bf(z["embed"]), "layers": layers, "norm": _bf(z["norm"]),
              "lm_head": _bf(z["lm_head"])}
    cache = {"k": [_bf(z[f"k_in{li}"]).copy() for li in range(2)],
             "v": [_bf(z[f"v_in{li}"]).copy() for li in range(2)]}
    logits = decoder.decode_step(params, z["tokens"][:, 0], cache, int(z["ctx"]), cfg)
    want = z["logits"]
    rms = np.sqrt(np.mean(want.astype(np.float64) ** 2))
    # bf16 activations through two layers: the two runs round at slightly
    # different sums; the acceptance figure is max-abs error over RMS
    assert np.max(np.abs(logits - want)) <= 2e-2 * rms
    assert np.array_equal(np.argmax(logits, -1), np.argmax(want, -1))
    for li in range(2):
        kd = np.abs(cache["k"][li].astype(np.float32) - _bf(z[f"k_out{li}"]).astype(np.float32))
        vd = np.abs(cache["v"][li].astype(np.float32) - _bf(z[f"v_out{li}"]).astype(np.float32))
        assert kd.max() <= 0.05 and vd.max() <= 0.05
        # untouched slots stay bit-identical
        ctx = int(z["ctx"])
        assert np.array_equal(cache["k"][li][:, :, :ctx].view(np.uint16), z[f"k_in{li}"][:, :, :ctx])
