"""Host-side logic of multi-GPU runs: one process per GPU, no data-path collective.

The decode path shards by independent sequences (replicas of the weights), so ranks only meet to
start together and to agree on the slowest rank's time; torch.distributed carries those two steps
(NCCL on GPUs, gloo in the CPU tests).
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
