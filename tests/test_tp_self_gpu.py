"""The tensor-parallel code path on ONE GPU: a group of one rank makes the decoder push its o / down
partial sums as {value, exchange number} lines into its own exchange block and form the sums in the
next projection's staging (once per rank, the result published to the other CTAs), and the pull
kernel and the NCCL path run against a world of one.  Same oracle, same
bound as the unsharded decoder; exercises the exchange builds of the kernels where no second GPU
is visible."""
import numpy as np
import pytest

from oracle import decoder as odec
from oracle import inputs
from util import dev, dev_params, host, pkg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["push", "pull", "nccl"])
@pytest.mark.parametrize("hidden,B", [(256, 3), (512, 1), (512, 2)])
def test_group_of_one_rank_takes_the_exchange_path(mode, hidden, B, monkeypatch):
    import torch
    p = pkg()
    from metal_pjrt_plugin_b200 import parallel
    monkeypatch.setenv("B200_TP_PUSH_ROWS", "8")
    if mode == "pull":
        monkeypatch.setenv("B200_TP_PULL", "1")
    else:
        monkeypatch.delenv("B200_TP_PULL", raising=False)
    ctx = p.Context(0)
    tp = parallel.TensorParallel.single(ctx)
    if mode != "nccl":
        tp.connect_peers(4 * hidden)
    cfg = inputs.decoder_config(layers=3, hidden=hidden, heads=4, kv_heads=2, head_dim=64, inter=2 * hidden, vocab=1024)
    ctxlen, max_len = 40, 64
    params, cache, tokens = inputs.config5(cfg, B, ctxlen, max_len=max_len)
    dec = p.qwen3.Decoder(dev_params(params), {k: [dev(a) for a in v] for k, v in cache.items()}, cfg, max_batch=B, ctx=ctx, tp=tp)
    try:
        tok = dev(tokens.astype(np.int32))
        pos = torch.tensor([ctxlen], dtype=torch.int32, device="cuda")
        logits = dec.step(tok, pos)
        first = logits.clone()
        for _ in range(10):          # many exchanges: slots and numbers keep alternating; the graph replays
            logits = dec.step(tok, pos)
        torch.cuda.synchronize()
        assert ctx.error() == 0
        assert torch.equal(first, logits)
        got = host(logits).reshape(B, -1)
    finally:
        dec.close()
        tp.close()
        ctx.close()
    want = odec.decode_step(params, tokens, {k: [a.copy() for a in v] for k, v in cache.items()}, ctxlen, cfg)
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    err = np.abs(got.astype(np.float64) - want) / rms
    assert np.mean(err <= 2e-2) >= 0.95 and err.max() <= 6e-2
    assert np.array_equal(got.argmax(-1), want.argmax(-1))
