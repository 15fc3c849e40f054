"""Tensor-parallel sharding arithmetic with world_size-2 gloo ranks on CPU: each rank
evaluates its shard of a decoder layer's projections with the NumPy oracle, the partial
sums meet in an all-reduce / all-gather, and the result equals the unsharded oracle.
This exercises parallel.py (row indices of the fused qkv / gate_up matrices, local
configs) exactly as bench.py and the GPU path use it.  No GPU, no library compute."""
import os
import sys

import numpy as np
import pytest

from util import ROOT, bf16, pkg


def _worker(rank, world, port, out_q):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from oracle import inputs, quant
    from __graft_entry__ import load_package
    load_package()
    from metal_pjrt_plugin_b200 import parallel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torch
    cfg = inputs.decoder_config(layers=1, hidden=128, heads=4, kv_heads=2, head_dim=64, inter=256, vocab=512)
    params, _, _ = inputs.config5(cfg, batch=2, ctx=4, max_len=8)   # same seed on every rank
    lp = params["layers"][0]
    x = np.random.default_rng(7).standard_normal((2, 128), dtype=np.float32).astype(bf16)
    local = parallel.local_config(cfg, world)
    assert local["heads"] == 2 and local["kv_heads"] == 1 and local["inter"] == 128 and local["vocab"] == 256

    def rows(w, idx):
        return {k: v[idx] for k, v in w.items()}

    def cols(w, sl):   # input columns [sl) of a [N, K] int4 matrix: words and groups
        return {"q4": w["q4"][:, sl.start // 8:sl.stop // 8], "s": w["s"][:, sl.start // 64:sl.stop // 64],
                "b": w["b"][:, sl.start // 64:sl.stop // 64]}

    def lin(xv, w, out=np.float32):
        return quant.qmm(xv, quant.bl_unpack_int4(w["q4"]), w["s"], w["b"], out)

    # qkv: output rows by head; the gathered result equals the full product row-permuted
    idx = parallel.qkv_row_index(cfg, rank, world)
    part = lin(x, rows(lp["qkv"], idx))
    gathered = [torch.zeros(part.shape) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(part))
    full = lin(x, lp["qkv"])
    all_idx = np.concatenate([parallel.qkv_row_index(cfg, r, world) for r in range(world)])
    ok_qkv = np.array_equal(np.concatenate([g.numpy() for g in gathered], axis=1), full[:, all_idx])
    assert sorted(all_idx.tolist()) == list(range(full.shape[1]))
    # o: input columns; f32 partial sums all-reduced equal the full product
    HD = cfg["heads"] * cfg["head_dim"]
    a = np.random.default_rng(8).standard_normal((2, HD), dtype=np.float32).astype(bf16)
    sl = parallel.shard_rows(HD, rank, world)
    po = torch.from_numpy(lin(a[:, sl], cols(lp["o"], sl)))
    dist.all_reduce(po)
    ok_o = np.allclose(po.numpy(), lin(a, lp["o"]), rtol=1e-5, atol=1e-5)
    # gate_up rows + down columns
    gidx = parallel.gate_up_row_index(cfg, rank, world)
    gu = lin(x, rows(lp["gate_up"], gidx), bf16)
    ok_gu = np.array_equal(gu.view(np.uint16), lin(x, lp["gate_up"], bf16)[:, gidx].view(np.uint16))
    out_q.put((rank, bool(ok_qkv), bool(ok_o), bool(ok_gu)))
    dist.destroy_process_group()


def test_sharded_projections_match_unsharded_world2():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p_ in procs:
        p_.start()
    res = [q.get(timeout=240) for _ in range(2)]
    for p_ in procs:
        p_.join(timeout=60)
        assert p_.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] and r[2] and r[3] for r in res), res


def test_local_config_rejects_uneven_shards():
    pkg()
    from metal_pjrt_plugin_b200 import parallel
    with pytest.raises(ValueError):
        parallel.local_config(dict(heads=32, kv_heads=8, inter=12288, vocab=151936), 3)
    assert parallel.shard_rows(4096, 3, 8) == slice(1536, 2048)
