"""Parity on the benchmarked workload itself: the full Qwen3-8B-shaped int4-g64 decoder
(36 layers, hidden 4096, 32 query / 8 KV heads of 128, intermediate 12288, vocabulary
151936 with an untied bf16 LM head) at position 2048 over a 2048-token cache, one step on
the GPU against the C restatement of the reference's forward (oracle/cpu_ref.c, all host
cores) on the same weights and cache.

What is asserted, and why not one number.  Per operator the bound for bf16 outputs is
max |error| <= 2e-2 x RMS(reference).  A decoder is a chain: every layer rounds its
activations to bf16, two correct evaluations round a few of them differently, and with
random-init weights (no trained structure to damp it) those flips grow from layer to layer.
So the test walks the depth: the same model cut to 1, 2, 4, 12 and all 36 layers.  With
one layer the per-operator bound itself must hold for 99.9 % of the 2 x 151936 logits and
no logit may be off by more than twice the bound (the LM head multiplies a hidden state in
which a handful of bf16 values differ by one ulp: over 300 000 logits the largest of the
resulting shifts reaches 2.4e-2 to 2.8e-2 x RMS; measured); for every depth the measured
error is printed; at full depth the test asserts what the reference's own model-level check asserts
of a bf16 run against its f32 CPU run (examples/llm/check.py:63-79,122): the same argmax
and KL(reference || this) < 0.05 per sequence, plus a ceiling on the measured error
(0.35 x RMS; 0.23 measured) so that a real regression still trips it."""
import numpy as np
import pytest

from util import host, pkg

pytestmark = pytest.mark.gpu

BATCH = 2
DEPTHS = (1, 2, 4, 12, 36)


@pytest.fixture(scope="module")
def full_model():
    import torch
    import bench
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
            hl[k] = {"q4": host(v["q4"]).view(np.uint32), "s": host(v["s"]), "b": host(v["b"])} if isinstance(v, dict) else host(v)
        hparams["layers"].append(hl)
    hcache = {k: [host(t).copy() for t in v] for k, v in cache.items()}
    return p, cfg, params, cache, tokens, hparams, hcache


def _log_softmax(x):
    x = x.astype(np.float64)
    x = x - x.max(-1, keepdims=True)
    return x - np.log(np.exp(x).sum(-1, keepdims=True))


def _oracle(full_model, depth):
    import bench
    from oracle import cpu_ref
    p, cfg, params, cache, tokens, hparams, hcache = full_model
    sub = dict(hparams, layers=hparams["layers"][:depth])
    c = {k: [a.copy() for a in v[:depth]] for k, v in hcache.items()}
    want = cpu_ref.decode_step(sub, tokens.numpy(), c, bench.CTX, dict(cfg, layers=depth))
    return want, c


@pytest.mark.parametrize("path", ["per_op", "stream"])
def test_full_size_step_against_the_cpu_restatement(full_model, path, monkeypatch):
    import torch
    import bench
    p, cfg, params, cache, tokens, hparams, hcache = full_model
    if path == "stream":
        monkeypatch.setenv("B200_DECODER_STREAM", "1")
    else:
        monkeypatch.delenv("B200_DECODER_STREAM", raising=False)
    errs = {}
    for depth in DEPTHS:
        want, ocache = _oracle(full_model, depth)
        sub_params = dict(params, layers=params["layers"][:depth])
        # every depth starts from the same cache contents: slot CTX is rewritten with the same values
        sub_cache = {k: v[:depth] for k, v in cache.items()}
        dec = p.qwen3.Decoder(sub_params, sub_cache, dict(cfg, layers=depth), max_batch=BATCH)
        logits = dec.step(tokens.to("cuda"), torch.tensor([bench.CTX], dtype=torch.int32, device="cuda"))
        torch.cuda.synchronize()
        assert p.default_context(0).error() == 0
        assert (dec.launches_per_step(BATCH) == 1) == (path == "stream")
        got = logits.cpu().numpy()
        rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        err = float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64))) / rms)
        lr, lp = _log_softmax(want), _log_softmax(got)
        kl = np.sum(np.exp(lr) * (lr - lp), -1)
        same = bool(np.array_equal(got.argmax(-1), want.argmax(-1)))
        errs[depth] = err
        print(f"full-size decoder ({path}), {depth:2d} layers: max logit error {err:.3e} x RMS, "
              f"KL(ref || got) max {kl.max():.2e}, argmax equal: {same}")
        if depth == 1:
            inside = float(np.mean(np.abs(got - want) <= 2e-2 * rms))
            print(f"    {100 * inside:.4f} % of the logits within 2e-2 x RMS")
            assert inside >= 0.999 and err <= 4e-2
        assert same and kl.max() < 0.05
        if depth == DEPTHS[-1]:
            assert err <= 0.35
            for li, tol in ((0, 8e-2), (17, 0.35), (35, 0.35)):   # the cache rows written this step (deeper: compounded)
                k = host(cache["k"][li])[:, :, bench.CTX].astype(np.float32)
                kw = ocache["k"][li][:, :, bench.CTX].astype(np.float32)
                assert np.max(np.abs(k - kw)) <= tol * float(np.sqrt(np.mean(kw * kw)))
        dec.close()
    print(f"error growth with depth ({path}): " + ", ".join(f"{d}: {e:.2e}" for d, e in errs.items()))
