"""Status codes and the sticky-error model on a real device
(≙ tests/test_gpu_errors.py:21-65 of the reference: an injected failure
surfaces, stays sticky, and nothing hangs).  Failures are made on the host;
no kernel is ever made to fault."""
import numpy as np
import pytest

from util import dev, pkg

pytestmark = pytest.mark.gpu


def test_injected_launch_failure_is_sticky():
    import torch
    p = pkg()
    ctx = p.Context(0)
    x = torch.randn(4, 64, device="cuda")
    p.rows.softmax(x, ctx=ctx)
    assert ctx.error() == 0
    before = ctx.launch_count
    ctx.fail_launch_after(2)
    p.rows.softmax(x, ctx=ctx)                       # launch 1 passes
    with pytest.raises(p.B200Error) as e:            # launch 2 is refused before it is enqueued
        p.rows.softmax(x, ctx=ctx)
    assert e.value.status == p._lib.INTERNAL and "injected" in str(e.value)
    assert ctx.launch_count == before + 1
    with pytest.raises(p.B200Error) as e2:           # sticky: every later call returns it
        p.rows.softmax(x, ctx=ctx)
    assert e2.value.status == p._lib.INTERNAL
    assert ctx.error() == p._lib.INTERNAL
    torch.cuda.synchronize()                         # the device itself is fine
    fresh = p.Context(0)
    y = p.rows.softmax(x, ctx=fresh)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all() and fresh.error() == 0


def test_invalid_arguments_do_not_poison_the_context():
    import torch
    p = pkg()
    ctx = p.Context(0)
    x = torch.randn(4, 64, device="cuda")
    with pytest.raises(p.B200Error) as e:
        p.rows.rownorm(9, x, ctx=ctx)
    assert e.value.status == p._lib.INVALID_ARGUMENT
    assert ctx.error() == 0
    p.rows.softmax(x, ctx=ctx)
    torch.cuda.synchronize()
    assert ctx.error() == 0


def test_bad_device_ordinal():
    p = pkg()
    with pytest.raises(p.B200Error) as e:
        p.Context(1000)
    assert e.value.status == p._lib.INVALID_ARGUMENT


def test_a_bounded_wait_that_runs_out_turns_into_a_sticky_timeout():
    """A device-side wait with a short limit on a barrier nobody arrives at: the kernel gives up
    and returns, the status word carries B200_TIMEOUT and the wait's id, the context's error is
    sticky, and a fresh context on the same device works.  Nothing faults or hangs."""
    import torch
    p = pkg()
    L, lib = p._lib, p.lib()
    ctx = p.Context(0)
    p._lib.check(lib.b200_context_wait_probe(ctx.handle, L.current_stream(), 200000))   # ~0.1 ms
    torch.cuda.synchronize()
    assert ctx.error() == L.TIMEOUT
    msg = lib.b200_last_error()
    assert b"TIMEOUT" in msg and b"900" in msg
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    st = lib.b200_rownorm(ctx.handle, L.current_stream(), 1, x.data_ptr(), None, None, x.data_ptr(), 4, 64, L.BF16, 1e-6)
    assert st == L.TIMEOUT                                   # sticky: every later call on this context returns it
    assert ctx.error() == L.TIMEOUT
    fresh = p.Context(0)
    p._lib.check(lib.b200_rownorm(fresh.handle, L.current_stream(), 1, x.data_ptr(), None, None, x.data_ptr(), 4, 64,
                                  L.BF16, 1e-6))
    torch.cuda.synchronize()
    assert fresh.error() == 0
    assert lib.b200_context_wait_probe(fresh.handle, L.current_stream(), 0) == L.INVALID_ARGUMENT
    fresh.close()
    ctx.close()


def test_umma_rate_probe_runs_and_reports_a_sane_cost():
    """The tcgen05.mma cost probe: runs, leaves the status word clean, and gives a per-instruction
    cost of the order the design notes quote (about 194 cycles; anything from 16 to 2000 passes,
    the test is about the plumbing, the number is for opbench)."""
    import torch
    p = pkg()
    ctx = p.Context(0)
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    for kind, m, n, at, nd in [(0, 128, 16, 1, 2), (1, 128, 256, 0, 1), (0, 64, 8, 0, 8)]:
        p._lib.check(p.lib().b200_probe_umma_rate(ctx.handle, p._lib.current_stream(), kind, m, n, at, nd, 128, out.data_ptr()))
        torch.cuda.synchronize()
        issue, done = (int(v) for v in out.tolist())
        assert 16 * 128 <= done <= 2000 * 128 and issue <= done
    assert ctx.error() == 0
    assert p.lib().b200_probe_umma_rate(ctx.handle, p._lib.current_stream(), 0, 128, 24, 1, 1, 16, out.data_ptr()) == p._lib.INVALID_ARGUMENT
