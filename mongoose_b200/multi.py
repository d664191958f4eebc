"""Host-side logic of multi-GPU runs: one process per GPU.

Two ways to use several GPUs.  Independent sequences (replicas of the weights) need no data-path
collective: ranks only meet to start together and to agree on the slowest rank's time, and
torch.distributed carries those two steps (NCCL on GPUs, gloo in the CPU tests).  Tensor
parallelism splits one model over the ranks; its exchanges run inside the C library on its own
NCCL communicator, and this module only computes partitions and hands the communicator id round.
"""
from __future__ import annotations

import os


def rank_env():
    """(rank, world_size, local_rank) as set by torchrun; (0, 1, 0) for a plain launch."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def sequences_for_rank(n_sequences: int, rank: int, world: int) -> list[int]:
    """Sequence i runs on GPU i mod G."""
    return [i for i in range(n_sequences) if i % world == rank]


def reduce_max(values, dist=None, device="cpu"):
    """Element-wise maximum over ranks of a list of floats (identity without a process group)."""
    import torch
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def aggregate_rate(world: int, units_per_rank: float, ms_max: float) -> float:
    """Whole-job throughput: every rank processed units_per_rank units in at most ms_max."""
    return world * units_per_rank / (ms_max / 1e3)


# -- tensor parallelism ------------------------------------------------------------------------
def tp_partition(cfg, rank: int, size: int) -> dict:
    """The part of the model rank `rank` of `size` holds (mg_tp_partition; host arithmetic only).
    Raises ValueError when the head counts cannot be split over `size` ranks."""
    import ctypes as C
    from . import _lib
    lib = _lib.load()
    c = _lib.MgConfig(dim=cfg.dim, kv_dim=cfg.kv_dim, head_dim=cfg.head_dim, n_heads=cfg.n_heads,
                      n_kv_heads=cfg.n_kv_heads, ffn_dim=cfg.ffn_dim, vocab=cfg.vocab, n_layers=cfg.n_layers,
                      max_seq=cfg.max_seq, rope_theta=float(cfg.rope_theta), rms_eps=float(cfg.eps),
                      layer_fmt=cfg.layer_fmt, head_fmt=cfg.head_fmt, device=0, max_batch=1, flags=0)
    out = _lib.MgTpShard()
    rc = lib.mg_tp_partition(C.byref(c), rank, size, C.byref(out))
    if rc != 0:
        raise ValueError(f"{cfg.name}: no tensor-parallel partition for rank {rank} of {size} (status {rc})")
    return {"q_heads": (out.q_head0, out.q_head1), "kv_heads": (out.kv_head0, out.kv_head1),
            "ffn": (out.ffn0, out.ffn1), "vocab": (out.vocab0, out.vocab1)}


def tp_unique_id() -> bytes:
    """A fresh 128-byte communicator id (rank 0 calls this)."""
    import ctypes as C
    from . import _lib
    buf = C.create_string_buffer(128)
    rc = _lib.load().mg_tp_unique_id(buf, 128)
    if rc != 0:
        raise RuntimeError(f"mg_tp_unique_id: status {rc}")
    return buf.raw


def share_unique_id(dist, rank: int) -> bytes:
    """Rank 0 makes the communicator id; every rank returns it (broadcast over `dist`)."""
    box = [tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    return box[0]
