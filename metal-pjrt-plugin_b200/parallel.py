"""Tensor-parallel group and weight sharding for the decoder (new: the
reference is single-device).  One process per GPU; torch.distributed moves the
128-byte NCCL id and nothing else."""
import ctypes as C

from . import _lib
from .context import default_context


class TensorParallel:
    def __init__(self, rank, world, id_bytes, ctx=None):
        import torch
        self.ctx = ctx or default_context(torch.cuda.current_device())
        self.rank, self.world = rank, world
        handle = C.c_void_p()
        buf = (C.c_char * _lib.TP_ID_BYTES).from_buffer_copy(id_bytes)
        _lib.check(_lib.lib().b200_tp_create(self.ctx.handle, buf, rank, world, C.byref(handle)))
        self.handle = handle
        self.peers_connected = False

    @staticmethod
    def make_id():
        buf = (C.c_char * _lib.TP_ID_BYTES)()
        _lib.check(_lib.lib().b200_tp_make_id(buf))
        return bytes(buf)

    @classmethod
    def from_torch_distributed(cls, ctx=None):
        """Rank 0 makes the id; torch.distributed broadcasts it."""
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        box = [cls.make_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return cls(rank, world, box[0], ctx)

    @classmethod
    def single(cls, ctx=None):
        """A group of one rank, made without torch.distributed.  A decoder created with it takes the
        sharded code path (push exchange, lines, two-level sum) on one GPU: for tests and profiles."""
        return cls(0, 1, cls.make_id(), ctx)

    def connect_peers(self, max_floats):
        """Allocates this rank's peer-exchange block (two slots of max_floats f32),
        gathers every rank's CUDA IPC handle over torch.distributed, maps the
        peers' blocks and synchronises the ranks.  After this the decoder's
        sums over ranks run as one kernel over peer memory instead of NCCL."""
        buf = (C.c_char * _lib.TP_PEER_HANDLE_BYTES)()
        _lib.check(_lib.lib().b200_tp_peer_alloc(self.handle, max_floats, buf))
        handles = [bytes(buf)]
        if self.world > 1:
            import torch.distributed as dist
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(buf))
        packed = (C.c_char * (_lib.TP_PEER_HANDLE_BYTES * self.world)).from_buffer_copy(b"".join(handles))
        _lib.check(_lib.lib().b200_tp_peer_connect(self.handle, packed))
        if self.world > 1:
            dist.barrier()
        self.peers_connected = True

    def peer_partial(self, slot, shape):
        """This rank's slot (0/1) of the exchange block as an f32 tensor view."""
        import torch
        ptr = _lib.lib().b200_tp_peer_partial(self.handle, slot)
        if not ptr:
            raise RuntimeError("peer exchange is not connected")
        iface = {"shape": tuple(shape), "typestr": "<f4", "data": (ptr, False), "version": 3}
        holder = type("PeerSlot", (), {"__cuda_array_interface__": iface})()
        return torch.as_tensor(holder, device=f"cuda:{self.ctx.device}")

    def sum_residual_norm(self, slot, x, gain, h, eps=1e-6, stream=None):
        """x += bf16(sum over ranks of slot), h = rms_norm(x) * gain (one kernel over peer memory)."""
        _lib.check(_lib.lib().b200_tp_sum_residual_norm(self.handle, stream or _lib.current_stream(), slot, _lib.ptr(x),
                                                        _lib.ptr(gain), _lib.ptr(h), x.shape[0], x.shape[1], eps))

    def all_reduce_bf16(self, t, stream=None):
        _lib.check(_lib.lib().b200_tp_all_reduce_bf16(self.handle, stream or _lib.current_stream(), _lib.ptr(t), t.numel()))

    def all_gather_f32(self, send, recv, stream=None):
        _lib.check(_lib.lib().b200_tp_all_gather_f32(self.handle, stream or _lib.current_stream(), _lib.ptr(send),
                                                     _lib.ptr(recv), send.numel()))

    def close(self):
        if self.handle:
            _lib.lib().b200_tp_destroy(self.handle)
            self.handle = None


def shard_rows(n, rank, world):
    """Contiguous block of n // world rows owned by `rank`."""
    per = n // world
    return slice(rank * per, (rank + 1) * per)


def local_config(cfg, world):
    """Per-rank head / intermediate / vocab counts."""
    for key in ("heads", "kv_heads", "inter", "vocab"):
        if cfg[key] % world:
            raise ValueError(f"{key}={cfg[key]} does not divide over {world} ranks")
    out = dict(cfg)
    out.update(heads=cfg["heads"] // world, kv_heads=cfg["kv_heads"] // world, inter=cfg["inter"] // world,
               vocab=cfg["vocab"] // world)
    return out


def qkv_row_index(cfg, rank, world):
    """Rows of the fused [q; k; v] matrix that rank owns (its query heads, its KV heads)."""
    import numpy as np
    H, KV, D = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    q = np.arange(H * D).reshape(world, -1)[rank]
    k = H * D + np.arange(KV * D).reshape(world, -1)[rank]
    v = (H + KV) * D + np.arange(KV * D).reshape(world, -1)[rank]
    return np.concatenate([q, k, v])


def gate_up_row_index(cfg, rank, world):
    import numpy as np
    inter = cfg["inter"]
    g = np.arange(inter).reshape(world, -1)[rank]
    return np.concatenate([g, inter + g])


def _contig(a):
    return a.contiguous() if hasattr(a, "contiguous") else __import__("numpy").ascontiguousarray(a)


def _rows(w, idx):
    if hasattr(idx, "dtype") and not isinstance(idx, slice) and hasattr(next(iter(w.values())), "device"):
        import torch
        idx = torch.as_tensor(idx, device=next(iter(w.values())).device)
    return {k: _contig(v[idx]) for k, v in w.items()}


def _cols(w, sl):
    """Input columns [sl) of an int4 [N, K] weight: K/8 words and K/64 groups per row."""
    return {"q4": _contig(w["q4"][:, sl.start // 8:sl.stop // 8]), "s": _contig(w["s"][:, sl.start // 64:sl.stop // 64]),
            "b": _contig(w["b"][:, sl.start // 64:sl.stop // 64])}


def shard_params(params, cache, cfg, rank, world):
    """This rank's shard of a decoder pytree (NumPy or torch): qkv and gate_up by output
    rows, o and down by input columns, the LM head by vocabulary rows, the KV cache by KV
    head; norms and the embedding are replicated.  Returns (params, cache, local cfg)."""
    local = local_config(cfg, world)
    D = cfg["head_dim"]
    hd = shard_rows(cfg["heads"] * D, rank, world)
    it = shard_rows(cfg["inter"], rank, world)
    kv = shard_rows(cfg["kv_heads"], rank, world)
    layers = []
    for lp in params["layers"]:
        layers.append({"attn_norm": lp["attn_norm"], "q_norm": lp["q_norm"], "k_norm": lp["k_norm"],
                       "mlp_norm": lp["mlp_norm"],
                       "qkv": _rows(lp["qkv"], qkv_row_index(cfg, rank, world)), "o": _cols(lp["o"], hd),
                       "gate_up": _rows(lp["gate_up"], gate_up_row_index(cfg, rank, world)),
                       "down": _cols(lp["down"], it)})
    out = {"embed": params["embed"], "norm": params["norm"], "layers": layers,
           "lm_head": _contig(params["lm_head"][shard_rows(cfg["vocab"], rank, world)])}
    lcache = {"k": [_contig(k[:, kv]) for k in cache["k"]], "v": [_contig(v[:, kv]) for v in cache["v"]]}
    return out, lcache, local
