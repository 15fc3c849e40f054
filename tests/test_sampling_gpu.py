"""b200_sample against the NumPy restatement of the reference's sample() (oracle/sampling.py):
greedy, temperature, top-k, top-k + top-p, ties, and the argument errors the reference raises."""
import numpy as np
import pytest

from oracle import sampling
from util import dev, host, pkg

pytestmark = pytest.mark.gpu


def _run(p, logits, u, **kw):
    import torch
    ld = dev(logits.astype(np.float32))
    ud = dev(u.astype(np.float32)) if u is not None else None
    out = p.qwen3.sample(ld, ud, **kw)
    torch.cuda.synchronize()
    return host(out)


@pytest.mark.parametrize("B,V", [(3, 1000), (2, 151936), (5, 4099)])
def test_greedy(B, V):
    p = pkg()
    rng = np.random.default_rng(1)
    logits = rng.standard_normal((B, V)).astype(np.float32) * 3
    logits[0, 7] = logits[0, V - 3] = logits[0].max() + 1       # a tie: the lower index wins
    got = _run(p, logits, None, temperature=0.0)
    want, _ = sampling.sample(logits, None, 0.0)
    assert np.array_equal(got, want) and got[0] == 7


@pytest.mark.parametrize("kw", [dict(temperature=0.8), dict(temperature=1.3, top_k=50), dict(temperature=0.7, top_k=1024),
                                dict(temperature=1.0, top_k=40, top_p=0.9), dict(temperature=0.5, top_k=200, top_p=0.5),
                                dict(temperature=2.0, top_k=1), dict(temperature=1.0, top_k=64, top_p=1e-6)])
@pytest.mark.parametrize("V", [2048, 151936])
def test_sampling_matches_the_oracle(kw, V):
    p = pkg()
    rng = np.random.default_rng(7)
    B = 24
    logits = (rng.standard_normal((B, V)) * 3).astype(np.float32)
    logits[1, :100] = logits[1, 100]                             # many equal values around the top-k boundary
    logits[2] = np.round(logits[2])                              # heavy ties everywhere
    u = rng.random(B).astype(np.float32)
    u[0], u[3] = 0.0, np.float32(1.0 - 2 ** -24)                 # the ends of the range
    got = _run(p, logits, u, **kw)
    want, margin = sampling.sample(logits, u.astype(np.float64), **kw)
    # draws whose target sits within f32 rounding of a CDF step may legitimately land on the neighbour
    sure = margin > 1e-4
    assert sure.sum() >= B // 2
    assert np.array_equal(got[sure], want[sure]), (kw, got, want)
    # every draw, sure or not, is one of the candidates the reference would keep
    if kw.get("top_k"):
        for r in range(B):
            z = logits[r].astype(np.float64)
            kth = np.sort(z)[::-1][kw["top_k"] - 1]
            assert z[got[r]] >= kth


def test_refusals():
    import torch
    p = pkg()
    L, lib = p._lib, p.lib()
    ctx = p.default_context()
    x = torch.zeros((2, 100), device="cuda")
    u = torch.zeros((2,), device="cuda")
    o = torch.zeros((2,), dtype=torch.int32, device="cuda")
    call = lambda t, k, pp, uu: lib.b200_sample(ctx.handle, L.current_stream(), x.data_ptr(), 2, 100, t, k, pp,
                                                uu.data_ptr() if uu is not None else None, o.data_ptr())
    assert call(-0.1, 0, 1.0, u) == L.INVALID_ARGUMENT and b"temperature" in lib.b200_last_error()
    assert call(1.0, 101, 1.0, u) == L.INVALID_ARGUMENT and b"top_k" in lib.b200_last_error()
    assert call(1.0, -1, 1.0, u) == L.INVALID_ARGUMENT
    assert call(1.0, 0, 0.9, u) == L.UNIMPLEMENTED
    assert call(1.0, 10, 0.9, None) == L.INVALID_ARGUMENT
    assert call(0.0, 0, 1.0, None) == L.OK
    assert ctx.error() == 0
