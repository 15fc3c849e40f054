"""Checkpoint loading (≙ Config.from_json / read_safetensors / load_params of the reference's
examples/llm/qwen3.py): the file format and the config rules on the CPU; the reference's
quantisers on the device, bit for bit against the NumPy restatement and the values recorded
from the reference itself; a synthetic checkpoint through load_params into one decode step."""
import json
import os
import struct

import numpy as np
import pytest

from oracle import decoder as odec
from oracle import quant
from util import bf16, dev, host, pkg

CFG = dict(model_type="qwen3", vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
           num_attention_heads=4, num_key_value_heads=2, head_dim=64, rope_theta=1e6, rms_norm_eps=1e-6,
           tie_word_embeddings=False, torch_dtype="bfloat16")


def write_safetensors(path, tensors):
    """A minimal writer of the published format: u64 header length, JSON header, raw data."""
    names = {np.dtype(bf16): "BF16", np.dtype(np.float16): "F16", np.dtype(np.float32): "F32"}
    header, blobs, off = {"__metadata__": {"format": "pt"}}, [], 0
    for k, a in tensors.items():
        raw = np.ascontiguousarray(a).tobytes()
        header[k] = {"dtype": names[a.dtype], "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def synthetic_checkpoint(root, cfg=CFG, seed=5):
    rng = np.random.default_rng(seed)
    E, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, KV, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    n = lambda *s: (0.05 * rng.standard_normal(s, dtype=np.float32)).astype(bf16)
    g = lambda d: (1 + 0.1 * rng.standard_normal(d, dtype=np.float32)).astype(bf16)
    t = {"model.embed_tokens.weight": n(V, E), "model.norm.weight": g(E), "lm_head.weight": n(V, E)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        t.update({p + "input_layernorm.weight": g(E), p + "post_attention_layernorm.weight": g(E),
                  p + "self_attn.q_proj.weight": n(H * D, E), p + "self_attn.k_proj.weight": n(KV * D, E),
                  p + "self_attn.v_proj.weight": n(KV * D, E), p + "self_attn.o_proj.weight": n(E, H * D),
                  p + "self_attn.q_norm.weight": g(D), p + "self_attn.k_norm.weight": g(D),
                  p + "mlp.gate_proj.weight": n(I, E), p + "mlp.up_proj.weight": n(I, E),
                  p + "mlp.down_proj.weight": n(E, I)})
    os.makedirs(root, exist_ok=True)
    keys = sorted(t)
    write_safetensors(os.path.join(root, "model-00001-of-00002.safetensors"), {k: t[k] for k in keys[:7]})
    write_safetensors(os.path.join(root, "model-00002-of-00002.safetensors"), {k: t[k] for k in keys[7:]})
    with open(os.path.join(root, "config.json"), "w") as f:
        json.dump(cfg, f)
    return t


def test_safetensors_round_trip(tmp_path):
    p = pkg()
    rng = np.random.default_rng(0)
    t = {"a": rng.standard_normal((3, 5), dtype=np.float32), "b.weight": rng.standard_normal((7,), dtype=np.float32).astype(bf16),
         "c": rng.standard_normal((2, 2, 4), dtype=np.float32).astype(np.float16), "empty": np.zeros((0, 4), np.float32)}
    write_safetensors(tmp_path / "x.safetensors", t)
    got = p.loader.read_safetensors(str(tmp_path / "x.safetensors"))
    assert set(got) == set(t)
    for k in t:
        assert got[k].dtype == t[k].dtype and got[k].shape == t[k].shape and got[k].tobytes() == t[k].tobytes()


def test_safetensors_refuses_other_dtypes(tmp_path):
    p = pkg()
    h = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    (tmp_path / "y.safetensors").write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 4)
    with pytest.raises(ValueError, match="F8_E4M3"):
        p.loader.read_safetensors(str(tmp_path / "y.safetensors"))


def test_config_from_json(tmp_path):
    p = pkg()

    def cfg_file(**kw):
        with open(tmp_path / "config.json", "w") as f:
            json.dump({**CFG, **kw}, f)
        return str(tmp_path / "config.json")

    c = p.loader.Config.from_json(cfg_file())
    assert (c.hidden_size, c.num_key_value_heads, c.tie_word_embeddings) == (256, 2, False)
    assert c.decoder_cfg() == dict(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=64, inter=512, vocab=512,
                                   theta=1e6, eps=1e-6)
    for bad in (dict(model_type="qwen3_moe"), dict(rope_scaling={"type": "yarn"}), dict(quantization_config={"x": 1})):
        with pytest.raises(ValueError):
            p.loader.Config.from_json(cfg_file(**bad))


@pytest.mark.gpu
def test_reference_int4_quantiser_on_the_device_matches_the_recorded_reference(golden_dir):
    import torch
    p = pkg()
    z = np.load(os.path.join(golden_dir, "quant_ref.npz"))
    got = p.loader.quantize_int4_ref(dev(z["w"]), layout="ref")
    torch.cuda.synchronize()
    assert np.array_equal(host(got["q4h"]), z["p4"])
    assert np.array_equal(host(got["s"]).view(np.uint16), z["s4"][..., 0].astype(bf16).view(np.uint16))
    assert np.array_equal(host(got["b"]).view(np.uint16), z["b4"][..., 0].astype(bf16).view(np.uint16))
    g8 = p.qwen3.quantize_int8(dev(z["w"]), 64)
    torch.cuda.synchronize()
    assert np.array_equal(host(g8["q"]), z["q8"].reshape(48, 256))
    assert np.array_equal(host(g8["s"]).view(np.uint16), z["s8"][..., 0].astype(bf16).view(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("N,K,kind", [(64, 128, "normal"), (1000, 4096, "normal"), (333, 1024, "edge"), (512, 12288, "bf16")])
def test_reference_int4_quantiser_bit_exact(N, K, kind):
    """Random weights, plus the grid's corner cases: all-zero and constant groups, groups
    whose largest magnitude is negative / positive, a zero edge, huge and tiny values."""
    import torch
    p = pkg()
    rng = np.random.default_rng(N + K)
    w = (0.02 * rng.standard_normal((N, K), dtype=np.float32))
    if kind == "edge":
        w[0] = 0
        w[1] = 0.37
        w[2] = -np.abs(w[2])
        w[3] = np.abs(w[3])
        w[4, :64] = np.linspace(-1, 0, 64)
        w[5, :64] = np.linspace(0, 1, 64)
        w[6] *= 1e30
        w[7] *= 1e-30
        w[8, ::64] = 3.0
        w[9, 5::64] = -3.0
    if kind == "bf16":
        w = w.astype(bf16)
    got = p.loader.quantize_int4_ref(dev(w), layout="ref")
    seq = p.loader.quantize_int4_ref(dev(w), layout="seq")
    torch.cuda.synchronize()
    pk, s, b = quant.ref_quantize_int4(w.astype(np.float32))
    assert np.array_equal(host(got["q4h"]), pk)
    assert np.array_equal(host(got["s"]).view(np.uint16), s[..., 0].astype(bf16).view(np.uint16))
    assert np.array_equal(host(got["b"]).view(np.uint16), b[..., 0].astype(bf16).view(np.uint16))
    assert np.array_equal(host(seq["q4"]).view(np.uint32), quant.split_half_to_seq(pk))


@pytest.mark.gpu
@pytest.mark.parametrize("quant_kind,layout", [("int4", "seq"), ("int4", "ref"), ("int8", "seq"), (None, "seq")])
def test_load_params_then_one_step(tmp_path, quant_kind, layout):
    """A synthetic two-shard checkpoint through load_params: the pytree has the reference's
    names and concatenations, the quantised matrices are the reference quantiser's, and (for
    the layout the decoder streams) one decode step agrees with the oracle on those weights."""
    import torch
    p = pkg()
    t = synthetic_checkpoint(str(tmp_path))
    cfg = p.loader.Config.from_json(str(tmp_path / "config.json"))
    params = p.loader.load_params(str(tmp_path), cfg, quant=quant_kind, layout=layout, block_rows=100)
    torch.cuda.synchronize()
    assert sorted(params) == ["embed", "layers", "lm_head", "norm"] and len(params["layers"]) == 2
    assert sorted(params["layers"][0]) == ["attn_norm", "down", "gate_up", "k_norm", "mlp_norm", "o", "q_norm", "qkv"]
    w = np.concatenate([t[f"model.layers.1.self_attn.{n}_proj.weight"] for n in "qkv"]).astype(np.float32)
    got = params["layers"][1]["qkv"]
    if quant_kind == "int4":
        pk, s, b = quant.ref_quantize_int4(w)
        if layout == "ref":
            assert np.array_equal(host(got["q4h"]), pk)
        else:
            assert np.array_equal(host(got["q4"]).view(np.uint32), quant.split_half_to_seq(pk))
        assert np.array_equal(host(got["s"]).view(np.uint16), s[..., 0].astype(bf16).view(np.uint16))
        assert np.array_equal(host(got["b"]).view(np.uint16), b[..., 0].astype(bf16).view(np.uint16))
    elif quant_kind == "int8":
        q, s = quant.ref_quantize_int8(w)
        assert np.array_equal(host(got["q"]), q.reshape(w.shape))
        assert np.array_equal(host(got["s"]).view(np.uint16), s[..., 0].astype(bf16).view(np.uint16))
    else:
        assert np.array_equal(host(got).view(np.uint16), w.astype(bf16).view(np.uint16))
    assert np.array_equal(host(params["lm_head"]).view(np.uint16), t["lm_head.weight"].view(np.uint16))
    # the projection through the public linear() on the loaded weight, against the oracle on the same bits
    x = (np.random.default_rng(3).standard_normal((3, 256), dtype=np.float32)).astype(bf16)
    y = p.qwen3.linear(dev(x), got)
    torch.cuda.synchronize()
    hw = {k: host(v) for k, v in got.items()} if isinstance(got, dict) else host(got)
    if isinstance(hw, dict) and "q4" in hw:
        hw["q4"] = hw["q4"].view(np.uint32)
    want = odec.linear(x, hw).astype(np.float32)
    rms = np.sqrt(np.mean(want ** 2))
    assert np.max(np.abs(host(y).astype(np.float32) - want)) <= 2e-2 * rms
    if quant_kind != "int4" or layout != "seq":
        return
    dcfg = cfg.decoder_cfg()
    B, ctx, S = 2, 9, 32
    cache = p.qwen3.init_cache(dcfg, B, S)
    hparams = {"embed": host(params["embed"]), "norm": host(params["norm"]), "lm_head": host(params["lm_head"]), "layers": []}
    for lp in params["layers"]:
        hl = {}
        for k, v in lp.items():
            hl[k] = {kk: (host(vv).view(np.uint32) if kk == "q4" else host(vv)) for kk, vv in v.items()} if isinstance(v, dict) else host(v)
        hparams["layers"].append(hl)
    ocache = {k: [host(a).copy() for a in v] for k, v in cache.items()}
    dec = p.qwen3.Decoder(params, cache, dcfg, max_batch=B)
    tok = np.array([5, 400], np.int32)
    logits = dec.step(dev(tok), torch.tensor([ctx], dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    want = odec.decode_step(hparams, tok.astype(np.int64), ocache, ctx, dcfg)
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    err = np.abs(host(logits).astype(np.float64) - want) / rms
    assert np.mean(err <= 2e-2) >= 0.95 and err.max() <= 6e-2
    assert np.array_equal(host(logits).argmax(-1), want.argmax(-1))
