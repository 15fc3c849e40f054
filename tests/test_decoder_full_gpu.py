"""Parity on the benchmarked workload itself: the full Qwen3-8B-shaped int4-g64 decoder
(36 layers, hidden 4096, 32 query / 8 KV heads of 128, intermediate 12288, vocabulary
151936 with an untied bf16 LM head) at position 2048 over a 2048-token cache, one step on
the GPU against the C restatement of the reference's forward (oracle/cpu_ref.c, all host
cores) on the same weights and cache.  Bound: max |logit error| <= 2e-2 x RMS(reference
logits) and the same argmax, as examples/llm/check.py:103-122 compares a run against the
f32 CPU run."""
import os

import numpy as np
import pytest

from util import dev, host, pkg

pytestmark = pytest.mark.gpu

BATCH = 2


@pytest.fixture(scope="module")
def full_model():
    import torch
    import bench
    from oracle import cpu_ref
    p = pkg()
    ctx = p.default_context(0)
    cfg = dict(bench.CFG)
    params, cache = bench.build_device_model(p, cfg, BATCH, "cuda:0", 4, 1, 0, ctx)
    g = torch.Generator(device="cpu")
    g.manual_seed(44)
    tokens = torch.randint(0, cfg["vocab"], (BATCH,), generator=g, dtype=torch.int32)
    # the same model on the host for the oracle
    hparams = {"embed": host(params["embed"]), "norm": host(params["norm"]), "lm_head": host(params["lm_head"]), "layers": []}
    for lp in params["layers"]:
        hl = {}
        for k, v in lp.items():
            if isinstance(v, dict):
                hl[k] = {"q4": host(v["q4"]).view(np.uint32), "s": host(v["s"]), "b": host(v["b"])}
            else:
                hl[k] = host(v)
        hparams["layers"].append(hl)
    hcache = {k: [host(t).copy() for t in v] for k, v in cache.items()}
    want = cpu_ref.decode_step(hparams, tokens.numpy(), hcache, bench.CTX, cfg)
    del hparams
    return p, cfg, params, cache, tokens, want, hcache


@pytest.mark.parametrize("path", ["stream", "per_op"])
def test_full_size_step_matches_the_cpu_restatement(full_model, path, monkeypatch):
    import torch
    import bench
    p, cfg, params, cache, tokens, want, hcache = full_model
    if path == "per_op":
        monkeypatch.setenv("B200_DECODER_NO_STREAM", "1")
    else:
        monkeypatch.delenv("B200_DECODER_NO_STREAM", raising=False)
    # each path starts from the same cache: slot CTX is rewritten with the same values by both
    dec = p.qwen3.Decoder(params, cache, cfg, max_batch=BATCH)
    logits = dec.step(tokens.to("cuda"), torch.tensor([bench.CTX], dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    assert p.default_context(0).error() == 0
    assert (dec.launches_per_step(BATCH) == 1) == (path == "stream")
    got = logits.cpu().numpy()
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    err = float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64))) / rms)
    same = bool(np.array_equal(got.argmax(-1), want.argmax(-1)))
    print(f"full-size decoder ({path}): max logit error {err:.3e} x RMS, argmax equal: {same}")
    assert err <= 2e-2
    assert same
    # the cache rows written this step
    for li in (0, 17, 35):
        k = host(cache["k"][li])[:, :, bench.CTX].astype(np.float32)
        kw = hcache["k"][li][:, :, bench.CTX].astype(np.float32)
        assert np.max(np.abs(k - kw)) <= 8e-2 * float(np.sqrt(np.mean(kw * kw)))
    dec.close()
