"""Weight-only quantised matmul on the device against the oracle: dequantised
tiles and nibble unpacking bit-exact, products within 2e-2 x RMS (bf16), the
device quantisers bit-exact, the reference-format fixture, edge cases."""
import os

import numpy as np
import pytest

from oracle import inputs, quant
from util import bf16, dev, host, pkg, rel_rms_err

pytestmark = pytest.mark.gpu
TOL = 2e-2  # max-abs error over RMS of the reference output, bf16 outputs


def _w4(packed, s, b):
    return {"q4": dev(packed), "s": dev(s), "b": dev(b)}


@pytest.mark.parametrize("n,k", [(64, 256), (48, 4096), (33, 64)])
def test_int4_dequant_bit_exact(n, k):
    import torch
    p = pkg()
    _, packed, s, b, _ = inputs.config4(1, k, n)
    want = quant.dequant_f32(quant.bl_unpack_int4(packed), s, b)
    got = host(p.qwen3.dequantize(_w4(packed, s, b), torch.float32))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    got16 = host(p.qwen3.dequantize(_w4(packed, s, b), torch.bfloat16))
    assert np.array_equal(got16.view(np.uint16), want.astype(bf16).view(np.uint16))


def test_int4_split_half_dequant_bit_exact(golden_dir):
    import torch
    p = pkg()
    z = np.load(os.path.join(golden_dir, "quant_ref.npz"))
    G = z["p4"].shape[1]
    s, b = z["s4"].astype(bf16).reshape(-1, G), z["b4"].astype(bf16).reshape(-1, G)
    w = {"q4h": dev(z["p4"]), "s": dev(s), "b": dev(b)}
    q = quant.ref_unpack_int4(z["p4"]).reshape(z["p4"].shape[0], -1)
    got = host(p.qwen3.dequantize(w, torch.float32))
    assert np.array_equal(got.view(np.uint32), quant.dequant_f32(q, s, b).view(np.uint32))


@pytest.mark.parametrize("group", [None, 64])
def test_int8_dequant_bit_exact(group):
    import torch
    p = pkg()
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((40, 512), dtype=np.float32) * 0.02).astype(np.float32)
    q, s = quant.bl_quantize_int8(w, group)
    got = host(p.qwen3.dequantize({"q": dev(q), "s": dev(s)}, torch.float32))
    assert np.array_equal(got.view(np.uint32), quant.dequant_f32(q, s, None).view(np.uint32))


def test_device_quantisers_bit_exact():
    p = pkg()
    rng = np.random.default_rng(6)
    w = (rng.standard_normal((96, 1024), dtype=np.float32) * 0.02).astype(np.float32)
    w[3, 64:128] = 0.0
    packed, s, b = quant.bl_quantize_int4(w)
    d = p.qwen3.quantize_int4(dev(w))
    assert np.array_equal(host(d["q4"]).view(np.uint32), packed)
    assert np.array_equal(host(d["s"]).view(np.uint16), s.view(np.uint16))
    assert np.array_equal(host(d["b"]).view(np.uint16), b.view(np.uint16))
    for group in (None, 64):
        q, s8 = quant.bl_quantize_int8(w, group)
        d8 = p.qwen3.quantize_int8(dev(w), group)
        assert np.array_equal(host(d8["q"]), q)
        assert np.array_equal(host(d8["s"]).view(np.uint16), s8.view(np.uint16))


@pytest.mark.parametrize("m", [1, 2, 3, 4, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("k,n", [(1024, 512), (4096, 1024)])
def test_int4_product(m, k, n):
    p = pkg()
    x, packed, s, b, _ = inputs.config4(m, k, n)
    want = quant.qmm(x, quant.bl_unpack_int4(packed), s, b, np.float32)
    got = host(p.qwen3.linear(dev(x), _w4(packed, s, b))).astype(np.float32)
    assert rel_rms_err(got, want) <= TOL


@pytest.mark.parametrize("m,k,n", [(1, 4096, 4096), (8, 4096, 12288), (32, 12288, 4096), (1, 12288, 4096),
                                   (32, 4096, 1024), (4, 12288, 4096), (5, 12288, 512), (16, 12288, 4096)])
def test_int4_product_qwen3_shapes(m, k, n):
    """Full Qwen3-8B projection shapes.  The CPU side checks a sample of the
    outputs (512 columns) so the suite stays fast."""
    p = pkg()
    x, packed, s, b, _ = inputs.config4(m, k, n)
    got = host(p.qwen3.linear(dev(x), _w4(packed, s, b))).astype(np.float32)
    cols = np.random.default_rng(0).choice(n, 512, replace=False)
    want = quant.qmm(x, quant.bl_unpack_int4(packed[cols]), s[cols], b[cols], np.float32)
    assert rel_rms_err(got[:, cols], want) <= TOL
    assert np.isfinite(got).all()


def test_int4_one_hot_rows_return_the_dequantised_column():
    """Size-independent property: with x = e_k the product is column k of the
    dequantised matrix (to bf16 rounding)."""
    p = pkg()
    k, n = 4096, 2048
    _, packed, s, b, _ = inputs.config4(1, k, n)
    ks = [0, 7, 63, 64, 1000, 4095]
    x = np.zeros((len(ks), k), np.float32)
    for i, kk in enumerate(ks):
        x[i, kk] = 1.0
    got = host(p.qwen3.linear(dev(x.astype(bf16)), _w4(packed, s, b))).astype(np.float32)
    wd = quant.dequant_f32(quant.bl_unpack_int4(packed), s, b)
    want = wd[:, ks].T
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(want), 1e-30))) - 7)
    assert np.all(np.abs(got - want) <= 0.51 * ulp + 1e-6)


def test_reference_format_against_fixture(golden_dir):
    """The reference's own int4 format (split-half bytes, MLX-style grid, possibly
    negative scale) and its _matvec_int4 output recorded from the reference."""
    p = pkg()
    z = np.load(os.path.join(golden_dir, "quant_ref.npz"))
    G = z["p4"].shape[1]
    # K = 256 here; pad nothing: the kernel takes any multiple of 64
    w = {"q4h": dev(z["p4"]), "s": dev(z["s4"].astype(bf16).reshape(-1, G)), "b": dev(z["b4"].astype(bf16).reshape(-1, G))}
    x = z["x"].view(bf16)
    got = host(p.qwen3.linear(dev(x), w)).astype(np.float32)
    want = z["mv4"].view(bf16).astype(np.float32)
    assert rel_rms_err(got, want) <= TOL
    # and the same values through the sequential layout
    seq = quant.split_half_to_seq(z["p4"])
    got2 = host(p.qwen3.linear(dev(x), {"q4": dev(seq), "s": w["s"], "b": w["b"]})).astype(np.float32)
    assert rel_rms_err(got2, want) <= TOL and rel_rms_err(got2, got) <= 1e-2  # same values, other k order
    # int8, group-wise (the reference's), against its _matvec_int8
    w8 = {"q": dev(z["q8"].reshape(z["q8"].shape[0], -1)), "s": dev(z["s8"].astype(bf16).reshape(-1, G))}
    got8 = host(p.qwen3.linear(dev(x), w8)).astype(np.float32)
    assert rel_rms_err(got8, z["mv8"].view(bf16).astype(np.float32)) <= TOL


@pytest.mark.parametrize("m", [1, 8, 32])
@pytest.mark.parametrize("k,n", [(4096, 1024), (1024, 4096)])
def test_int8_per_channel_product(m, k, n):
    p = pkg()
    x, q, s, _ = inputs.config3(m, k, n)
    want = quant.qmm(x, q, s, None, np.float32)
    got = host(p.qwen3.linear(dev(x), {"q": dev(q), "s": dev(s)})).astype(np.float32)
    assert rel_rms_err(got, want) <= TOL


@pytest.mark.parametrize("m", [1, 5, 32])
def test_bf16_weights_product(m):
    """bits = 16: the LM-head form (bf16 [out, in] matrix), f32 logits holding bf16-rounded values."""
    p = pkg()
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((1000, 512), dtype=np.float32) * 0.02).astype(bf16)
    x = rng.standard_normal((m, 512), dtype=np.float32).astype(bf16)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    got = host(p.qwen3.linear(dev(x), dev(w), out_f32=True))
    assert got.dtype == np.float32 and rel_rms_err(got, want) <= TOL
    assert np.array_equal(got, got.astype(bf16).astype(np.float32))  # values are bf16-representable


def test_edge_cases():
    import torch
    p = pkg()
    # ragged N (not a multiple of 16), smallest K, strided x, residual epilogue
    x, packed, s, b, _ = inputs.config4(3, 64, 37)
    want = quant.qmm(x, quant.bl_unpack_int4(packed), s, b, np.float32)
    w = _w4(packed, s, b)
    assert rel_rms_err(host(p.qwen3.linear(dev(x), w)).astype(np.float32), want) <= TOL
    xs = torch.zeros((3, 200), dtype=torch.bfloat16, device="cuda")
    xs[:, :64] = dev(x)
    assert np.array_equal(host(p.qwen3.linear(xs[:, :64], w)).view(np.uint16), host(p.qwen3.linear(dev(x), w)).view(np.uint16))
    res = np.random.default_rng(1).standard_normal((3, 37), dtype=np.float32).astype(bf16)
    got = host(p.qwen3.linear(dev(x), w, residual=dev(res))).astype(np.float32)
    want_r = (res.astype(np.float32) + want.astype(bf16).astype(np.float32)).astype(bf16).astype(np.float32)
    assert rel_rms_err(got, want_r) <= TOL
    # empty problems launch nothing
    n0 = p.default_context().launch_count
    out = p.qwen3.linear(dev(x)[:0], w)
    assert out.shape == (0, 37) and p.default_context().launch_count == n0
    # more than 32 rows with a fused input transform: refused, not wrong
    with pytest.raises(p.B200Error) as e:
        p.qwen3.linear(torch.zeros((33, 128), dtype=torch.bfloat16, device="cuda"), w, silu_mul=True)
    assert e.value.status == p._lib.UNIMPLEMENTED
    with pytest.raises(p.B200Error) as e:
        p.qwen3.linear(torch.zeros((33, 64), dtype=torch.bfloat16, device="cuda"), w, out_f32=True)
    assert e.value.status == p._lib.UNIMPLEMENTED
    assert p.default_context().error() == 0


def test_unaligned_inputs_take_the_general_variant():
    """K = 4096 with x (or the scales) off a 16-byte boundary: the unrolled variants assume
    16-byte loads, so the general one must be chosen, with the same result (to bf16 rounding)."""
    import torch
    p = pkg()
    x, packed, s, b, _ = inputs.config4(2, 4096, 4096)
    w = _w4(packed, s, b)
    ref = host(p.qwen3.linear(dev(x), w)).astype(np.float32)
    xo = torch.zeros((2, 4096 + 8), dtype=torch.bfloat16, device="cuda")
    xo[:, 1:4097] = dev(x)
    assert rel_rms_err(host(p.qwen3.linear(xo[:, 1:4097], w)).astype(np.float32), ref) <= 2e-3   # x two bytes off
    so = torch.zeros(s.size + 1, dtype=torch.bfloat16, device="cuda")
    so[1:] = dev(s).reshape(-1)
    w2 = dict(w, s=so[1:].reshape(s.shape))
    assert rel_rms_err(host(p.qwen3.linear(dev(x), w2)).astype(np.float32), ref) <= 2e-3          # scales two bytes off


@pytest.mark.parametrize("m", [1, 2, 3, 8])
@pytest.mark.parametrize("bits", [4, 16])
@pytest.mark.parametrize("n", [512, 4096])   # K split across a cluster (two-pass norm) / whole rows per CTA (one pass)
def test_fused_rmsnorm_prologue(m, bits, n):
    """linear(rms_norm(x, gain, eps), w) with the norm fused into the input staging."""
    from oracle import rownorm
    p = pkg()
    k = 1024
    x, packed, s, b, _ = inputs.config4(m, k, n)
    gain = (1 + 0.1 * np.random.default_rng(3).standard_normal(k, dtype=np.float32)).astype(bf16)
    h = rownorm.rms_norm(x, gain, 1e-6)
    if bits == 4:
        w = _w4(packed, s, b)
        want = quant.qmm(h, quant.bl_unpack_int4(packed), s, b, np.float32)
    else:
        wm = (np.random.default_rng(4).standard_normal((n, k), dtype=np.float32) * 0.02).astype(bf16)
        w = dev(wm)
        want = h.astype(np.float64) @ wm.astype(np.float64).T
    got = host(p.qwen3.linear(dev(x), w, rms_gain=dev(gain), eps=1e-6)).astype(np.float32)
    assert rel_rms_err(got, want) <= TOL
    # and it equals the two-kernel path to within bf16 rounding of h
    two = host(p.qwen3.linear(p.rows.rms_norm(dev(x), dev(gain), 1e-6), w)).astype(np.float32)
    assert rel_rms_err(got, two) <= TOL
    with pytest.raises(p.B200Error):
        import torch
        p.qwen3.linear(torch.zeros((9, k), dtype=torch.bfloat16, device="cuda"), w, rms_gain=dev(gain))


@pytest.mark.parametrize("m", [1, 8, 32])
def test_fused_silu_mul_prologue(m):
    """linear(silu(gate) * up, w) for x = [gate | up]."""
    from oracle import decoder as odec
    p = pkg()
    k, n = 1536, 256
    _, packed, s, b, _ = inputs.config4(1, k, n)
    gu = (np.random.default_rng(8).standard_normal((m, 2 * k), dtype=np.float32) * 1.5).astype(bf16)
    act = odec.silu_mul(gu[:, :k], gu[:, k:])
    want = quant.qmm(act, quant.bl_unpack_int4(packed), s, b, np.float32)
    got = host(p.qwen3.linear(dev(gu), _w4(packed, s, b), silu_mul=True)).astype(np.float32)
    assert got.shape == (m, n) and rel_rms_err(got, want) <= TOL


@pytest.mark.parametrize("m", [33, 64, 128, 512])
@pytest.mark.parametrize("fmt", ["int4", "int4_split_half", "int8_g64", "int8_channel", "bf16"])
def test_many_rows_go_through_dequantise_and_gemm(m, fmt):
    """More than 32 rows of x: panel-wise dequantisation into the L2-resident workspace + tensor-core
    GEMM, for every weight format, against the oracle; one shape spans several panels."""
    import torch
    p = pkg()
    k, n = (4096, 9000) if (fmt == "int4" and m == 64) else (1024, 520)   # 9000 rows x 4096: three panels, ragged tail
    rng = np.random.default_rng(m)
    x = rng.standard_normal((m, k), dtype=np.float32).astype(bf16)
    w = (0.02 * rng.standard_normal((n, k), dtype=np.float32))
    if fmt == "int4":
        packed, s, b = quant.bl_quantize_int4(w)
        wd, q = _w4(packed, s, b), quant.bl_unpack_int4(packed)
    elif fmt == "int4_split_half":
        pk, s3, b3 = quant.ref_quantize_int4(w)
        s, b = s3[..., 0].astype(bf16), b3[..., 0].astype(bf16)
        wd = {"q4h": dev(pk), "s": dev(s), "b": dev(b)}
        q = quant.ref_unpack_int4(pk).reshape(n, k)
    elif fmt.startswith("int8"):
        q, s = quant.bl_quantize_int8(w, 64 if fmt == "int8_g64" else None)
        b = None
        wd = {"q": dev(q), "s": dev(s)}
    else:
        wm = w.astype(bf16)
        wd = dev(wm)
    if fmt == "bf16":
        want = x.astype(np.float64) @ wm.astype(np.float64).T
    else:
        cols = np.random.default_rng(0).choice(n, 256, replace=False)
        want = quant.qmm(x, q[cols], s[cols], None if b is None else b[cols], np.float32)
    got = host(p.qwen3.linear(dev(x), wd)).astype(np.float32)
    torch.cuda.synchronize()
    assert got.shape == (m, n) and np.isfinite(got).all()
    assert rel_rms_err(got if fmt == "bf16" else got[:, cols], want) <= TOL
    if fmt == "int4":
        res = rng.standard_normal((m, n), dtype=np.float32).astype(bf16)
        got_r = host(p.qwen3.linear(dev(x), wd, residual=dev(res))).astype(np.float32)
        want_r = res.astype(np.float32)[:, cols] + want
        assert rel_rms_err(got_r[:, cols], want_r) <= TOL
    assert p.default_context().error() == 0


@pytest.mark.parametrize("m", [1, 8, 32])
@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 12288), (12288, 4096)])
def test_int8_per_channel_product_qwen3_shapes(m, k, n):
    """The int8 per-channel products of the benchmark configuration at full size (a sample of 512
    output channels is checked on the CPU)."""
    p = pkg()
    x, q, s, _ = inputs.config3(m, k, n)
    got = host(p.qwen3.linear(dev(x), {"q": dev(q), "s": dev(s)})).astype(np.float32)
    cols = np.random.default_rng(1).choice(n, 512, replace=False)
    want = quant.qmm(x, q[cols], s[cols], None, np.float32)
    assert rel_rms_err(got[:, cols], want) <= TOL
    assert np.isfinite(got).all()


def _one_hot_check(p, wd, dense, k, ks, m):
    """x row i = e_{ks[i]} (the other rows of the batch zero): the product is column ks[i] of the
    dequantised matrix, to the one bf16 rounding of the output."""
    x = np.zeros((m, k), np.float32)
    for i, kk in enumerate(ks):
        x[i, kk] = 1.0
    got = host(p.qwen3.linear(dev(x.astype(bf16)), wd)).astype(np.float32)
    want = np.zeros((m, dense.shape[0]), np.float32)
    want[:len(ks)] = dense[:, ks].T
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(want), 1e-30))) - 7)
    assert np.all(np.abs(got - want) <= 0.51 * ulp + 1e-6)


@pytest.mark.parametrize("m", [9, 17, 32])
@pytest.mark.parametrize("k", [4096, 12288])
def test_int4_one_hot_unpack_at_every_batch_block(m, k):
    """The nibble order and the k mapping of every batch-block variant (two, three and four blocks
    of 8 rows), K = 4096 and K = 12288 (the K-split forms): positions inside a word, across words,
    groups, copy chunks and K slices."""
    p = pkg()
    n = 1024
    _, packed, s, b, _ = inputs.config4(1, k, n)
    ks = [0, 1, 6, 7, 8, 63, 64, 65, 511, 512, 2047, 2048, k // 2 - 1, k // 2, k - 65, k - 64, k - 1][:m]
    dense = quant.dequant_f32(quant.bl_unpack_int4(packed), s, b)
    _one_hot_check(p, _w4(packed, s, b), dense, k, ks, m)


@pytest.mark.parametrize("m", [1, 8, 17])
def test_int4_split_half_one_hot_unpack(m):
    """The reference's split-half byte layout (element j in the low nibble of byte j, element j + 32
    in the high nibble) through the product kernel."""
    p = pkg()
    k, n = 4096, 512
    rng = np.random.default_rng(12)
    w = 0.02 * rng.standard_normal((n, k), dtype=np.float32)
    pk, s3, b3 = quant.ref_quantize_int4(w)
    s, b = s3[..., 0].astype(bf16), b3[..., 0].astype(bf16)
    wd = {"q4h": dev(pk), "s": dev(s), "b": dev(b)}
    dense = quant.dequant_f32(quant.ref_unpack_int4(pk).reshape(n, k), s, b)
    ks = [0, 1, 31, 32, 33, 63, 64, 95, 96, 127, 2048, 2079, 2080, 4032, 4063, 4064, 4095][:m]
    _one_hot_check(p, wd, dense, k, ks, m)


@pytest.mark.parametrize("group", [None, 64])
@pytest.mark.parametrize("m,k", [(1, 4096), (8, 12288), (17, 4096), (32, 12288)])
def test_int8_one_hot_unpack(group, m, k):
    p = pkg()
    n = 512
    rng = np.random.default_rng(13)
    w = 0.02 * rng.standard_normal((n, k), dtype=np.float32)
    q, s = quant.bl_quantize_int8(w, group)
    dense = quant.dequant_f32(q, s, None, group or k)
    ks = [0, 1, 15, 16, 63, 64, 127, 128, 1023, 1024, 2047, 2048, k // 2, k - 129, k - 128, k - 64, k - 1][:m]
    _one_hot_check(p, {"q": dev(q), "s": dev(s)}, dense, k, ks, m)


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("k,inter,fuse_norm", [(1024, 768, False), (1024, 768, True), (4096, 12288, True)])
def test_silu_pair_epilogue(m, k, inter, fuse_norm):
    """gate_up on its row-interleaved copy with silu(gate) * up formed in the projection's epilogue:
    equal to the two-step form (projection to bf16, then silu_mul) on the same weights."""
    from oracle import decoder as odec
    from oracle import rownorm
    p = pkg()
    x, packed, s, b, _ = inputs.config4(m, k, 2 * inter)
    w = _w4(packed, s, b)
    wp = p.qwen3.interleave_gate_up(w)
    gain = (1 + 0.1 * np.random.default_rng(3).standard_normal(k, dtype=np.float32)).astype(bf16)
    kw = dict(rms_gain=dev(gain), eps=1e-6) if fuse_norm else {}
    got = host(p.qwen3.linear(dev(x), wp, silu_pair=True, **kw))
    assert got.shape == (m, inter)
    # the device's own two-step form: same sums, same roundings
    gu = p.qwen3.linear(dev(x), w, **kw)
    two = host(gu).astype(np.float32)
    want_dev = odec.silu_mul(two[:, :inter].astype(bf16), two[:, inter:].astype(bf16))
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(want_dev.astype(np.float32)), 1e-30))) - 7)
    assert np.all(np.abs(got.astype(np.float32) - want_dev.astype(np.float32)) <= 1.01 * ulp)
    # and against the oracle end to end (a sample of columns at full size)
    cols = np.random.default_rng(0).choice(inter, min(inter, 256), replace=False)
    h = rownorm.rms_norm(x, gain, 1e-6) if fuse_norm else x
    rows = np.concatenate([cols, inter + cols])
    q = quant.bl_unpack_int4(packed[rows])
    gu_ref = quant.qmm(h, q, s[rows], b[rows], bf16)
    want = odec.silu_mul(gu_ref[:, :len(cols)], gu_ref[:, len(cols):]).astype(np.float32)
    assert rel_rms_err(got.astype(np.float32)[:, cols], want) <= 3e-2
    # the rows of the copy are the original's, rearranged
    qp = host(wp["q4"]).view(np.uint32)
    assert np.array_equal(qp[0:8], packed[0:8]) and np.array_equal(qp[8:16], packed[inter:inter + 8])
    assert np.array_equal(qp[16:24], packed[8:16])
