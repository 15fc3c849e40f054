"""Tensor-parallel decoder on 2 GPUs (one process per GPU, NCCL through the library)
against the unsharded CPU oracle.  Skipped where fewer than two devices are visible.
Ranks leave only after the step has been synchronised; NVLS is switched off for NCCL."""
import datetime
import os
import sys
import traceback

import numpy as np
import pytest

from util import ROOT

pytestmark = pytest.mark.gpu


def _guarded(body, rank, out_q, *args):
    """A rank that raises says so through the queue at once, so the test fails in seconds
    instead of waiting for its own limit."""
    try:
        body(rank, *args)
    except BaseException:
        out_q.put((rank, ("error", traceback.format_exc())))
        raise


def _worker(rank, world, port, out_q, peers, hidden, B):
    _guarded(_worker_body, rank, out_q, world, port, out_q, peers, hidden, B)


def _timeout_worker(rank, world, port, out_q):
    _guarded(_timeout_worker_body, rank, out_q, world, port, out_q)


def _collect(q, procs):
    res = {}
    for _ in procs:
        rank, r = q.get(timeout=200)
        if isinstance(r, tuple) and len(r) == 2 and r[0] == "error":
            for p_ in procs:
                p_.join(timeout=100)
            pytest.fail(f"rank {rank} raised:\n{r[1]}")
        res[rank] = r
    for p_ in procs:
        p_.join(timeout=120)
        assert p_.exitcode == 0
    return res


def _worker_body(rank, world, port, out_q, peers, hidden, B):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    if peers == "pull":   # the separate exchange kernel instead of the push from the projections' epilogue
        os.environ["B200_TP_PULL"] = "1"
    else:
        os.environ.pop("B200_TP_PULL", None)
        os.environ["B200_TP_PUSH_ROWS"] = "8"   # the push at every batch it supports (the default stops at 2 rows)
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from oracle import decoder as odec
    from oracle import dense, inputs
    from util import dev, dev_params, host
    from __graft_entry__ import load_package
    pkg = load_package()
    from metal_pjrt_plugin_b200 import parallel
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=90))
    ctx = pkg.Context(rank)
    tp = parallel.TensorParallel.from_torch_distributed(ctx)
    if peers:   # the sums over ranks over peer memory instead of NCCL
        tp.connect_peers(4 * hidden)
    cfg = inputs.decoder_config(layers=3, hidden=hidden, heads=4, kv_heads=2, head_dim=64, inter=2 * hidden, vocab=1024)
    ctxlen, max_len = 40, 64
    params, cache, tokens = inputs.config5(cfg, B, ctxlen, max_len=max_len)
    sp, sc, local = parallel.shard_params(params, cache, cfg, rank, world)
    device = f"cuda:{rank}"
    dp = dev_params(sp, device)
    dc = {k: [dev(a, device) for a in v] for k, v in sc.items()}
    dec = pkg.qwen3.Decoder(dp, dc, local, max_batch=B, ctx=ctx, tp=tp)
    tok = dev(tokens.astype(np.int32), device)
    pos = torch.tensor([ctxlen], dtype=torch.int32, device=device)
    logits = dec.step(tok, pos)
    logits2 = dec.step(tok, pos).clone()      # graph replay
    for _ in range(20):                       # many exchanges: the slots and flags keep alternating
        logits3 = dec.step(tok, pos)
    torch.cuda.synchronize()
    assert torch.equal(logits3, logits2)
    status = ctx.error()
    got = host(logits)                                           # [world, B, V / world], rank-major
    got = np.concatenate([got[r] for r in range(world)], axis=-1)
    res = None
    if rank == 0:
        want = odec.decode_step(params, tokens, {k: [a.copy() for a in v] for k, v in cache.items()}, ctxlen, cfg)
        res = (float(dense.max_abs_over_rms(got, want)), bool(np.array_equal(got.argmax(-1), want.argmax(-1))),
               bool(torch.equal(logits, logits2)), int(status))
    dist.barrier()
    out_q.put((rank, res))
    dec.close()
    tp.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("peers,hidden,B", [(False, 256, 3), ("pull", 256, 3), ("push", 256, 3), ("push", 512, 1),
                                            ("push", 512, 2), ("push", 256, 8), ("push", 256, 4)])
def test_tp2_decoder_matches_oracle(peers, hidden, B):
    """Sums over ranks by NCCL, by the exchange kernel that pulls the peers' partial sums, and by
    the projections pushing theirs (the two RMSNorm staging variants of the consuming
    projection: rows that fit one pass, and the two-pass form)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + {False: 0, "pull": 7, "push": 13}[peers] + hidden // 64 + B
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, peers, hidden, B)) for r in range(2)]
    for p_ in procs:
        p_.start()
    res = _collect(q, procs)
    err, same_argmax, replay_equal, status = res[0]
    assert status == 0
    print(f"tp2 {peers} hidden {hidden} batch {B}: max logit error {err:.3e} x RMS")
    assert err <= 6e-2 and same_argmax and replay_equal


def _timeout_worker_body(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    from metal_pjrt_plugin_b200 import parallel
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=90))
    ctx = pkg.Context(rank)
    tp = parallel.TensorParallel.from_torch_distributed(ctx)
    B, E = 2, 256
    tp.connect_peers(B * E)
    dev = f"cuda:{rank}"
    x = torch.ones((B, E), dtype=torch.bfloat16, device=dev)
    gain = torch.ones((E,), dtype=torch.bfloat16, device=dev)
    h = torch.empty_like(x)
    tp.peer_partial(0, (B, E)).fill_(0.5)
    tp.peer_partial(1, (B, E)).fill_(0.25)
    torch.cuda.synchronize()
    dist.barrier()
    tp.sum_residual_norm(0, x, gain, h)            # exchange 1: both ranks take part
    torch.cuda.synchronize()
    ok_first = bool(torch.all(x == 2.0).item()) and ctx.error() == 0     # 1 + 0.5 + 0.5
    dist.barrier()
    status, message = 0, ""
    if rank == 0:
        # exchange 2: the peer stays alive (it waits at the host barrier below) but never joins
        tp.sum_residual_norm(1, x, gain, h)
        torch.cuda.synchronize()                    # the wait runs out after about two seconds; the kernel returns
        status = ctx.error()
        message = pkg.lib().b200_last_error().decode()
        untouched = bool(torch.all(x == 2.0).item())     # nothing was summed, nothing written
    else:
        untouched = True
    dist.barrier()                                  # both ranks leave together, with nothing in flight
    out_q.put((rank, (ok_first, status, message, untouched)))
    tp.close()
    dist.destroy_process_group()


def test_tp2_exchange_wait_runs_out_when_a_peer_skips_an_exchange():
    """Rank 1 stays alive but skips one exchange: rank 0's bounded wait for its flag expires,
    the kernel reads nothing of the peer, writes nothing, reports B200_TIMEOUT with the peer's
    wait id, and both ranks then tear down normally.  No GPU faults or hangs."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from util import pkg
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000 + 101
    procs = [ctx.Process(target=_timeout_worker, args=(r, 2, port, q)) for r in range(2)]
    for p_ in procs:
        p_.start()
    res = _collect(q, procs)
    TIMEOUT = pkg()._lib.TIMEOUT
    ok_first, status, message, untouched = res[0]
    assert ok_first and res[1][0]
    assert status == TIMEOUT and "401" in message and untouched
    assert res[1][1] == 0
