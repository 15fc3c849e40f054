"""The attention entry point that allocates nothing (b200_attention_decode_static).

It exists for callers that are not allowed to allocate device memory at the call site:
code running inside a stream capture, or a host runtime whose allocator owns the whole
device.  Its split-attention partials live in a fixed array inside the library instead of
a caller buffer.  Here it is called through the C ABI twice in a row, on different inputs,
and each result is compared with the ordinary entry point (caller-provided scratch) on the
same inputs; the second call also shows that what the first call left in the shared array
does not leak into the next result.  Collected last on purpose."""
import numpy as np
import pytest

from util import bf16, dev, host, pkg, rel_rms_err

pytestmark = pytest.mark.gpu


def _inputs(seed, B, H, KV, D, S, pos):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, H, D), dtype=np.float32).astype(bf16)
    kc = rng.standard_normal((B, KV, S, D), dtype=np.float32).astype(bf16)
    vc = rng.standard_normal((B, KV, D, S), dtype=np.float32).astype(bf16)
    return q, kc, vc, pos


def test_static_scratch_attention_matches_the_allocating_entry_point_twice():
    import torch
    p = pkg()
    L = p.lib()
    ctx = p.default_context()
    stream = p._lib.current_stream()
    B, H, KV, D, S = 2, 8, 2, 128, 320
    for seed, pos in ((1, 319), (2, 70)):          # two calls in a row; the second attends fewer slots
        q, kc, vc, pos = _inputs(seed, B, H, KV, D, S, pos)
        qd, kd, vd = dev(q), dev(kc), dev(vc)
        posd = torch.tensor([pos], dtype=torch.int32, device="cuda")
        want = torch.empty((B, H, D), dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(L.b200_attention_scratch_bytes(B, H, D, S) // 4, device="cuda")
        p._lib.check(L.b200_attention_decode(ctx.handle, stream, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(),
                                             want.data_ptr(), posd.data_ptr(), scratch.data_ptr(), B, H, KV, D, S))
        got = torch.full((B, H, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        p._lib.check(L.b200_attention_decode_static(ctx.handle, stream, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(),
                                                    got.data_ptr(), posd.data_ptr(), B, H, KV, D, S))
        torch.cuda.synchronize()
        g, w = host(got).astype(np.float32), host(want).astype(np.float32)
        assert np.isfinite(g).all()
        assert rel_rms_err(g, w) <= 2e-2          # the tolerance the other attention tests use
        assert np.array_equal(g, w)               # and in fact the same kernels ran: the same bits
    assert ctx.error() == 0


def test_static_scratch_refuses_what_does_not_fit():
    import torch
    p = pkg()
    L = p.lib()
    ctx = p.default_context()
    t = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    posd = torch.zeros(1, dtype=torch.int32, device="cuda")
    # 32 sequences x 32 heads x 32768 slots of partials is far beyond 8 MiB
    st = L.b200_attention_decode_static(ctx.handle, p._lib.current_stream(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                        t.data_ptr(), posd.data_ptr(), 32, 32, 8, 128, 32768)
    assert st == p._lib.RESOURCE_EXHAUSTED
    assert b"8388608" in L.b200_last_error() and ctx.error() == 0
