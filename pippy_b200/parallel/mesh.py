"""Process-group layout for composing pipeline, data, tensor and expert parallelism.

Ranks are laid out with the tensor/expert dimension fastest, then pipeline, then data:
``global = (dp * pp_size + pp) * tp_size + tp``, so the ranks of one tensor-parallel group are neighbours
(the reference composes with ``DeviceMesh`` sub-groups the same way, test/test_composability.py:130-151).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch.distributed as dist


@dataclass
class ParallelMesh:
    pp_size: int
    dp_size: int
    tp_size: int
    pp_rank: int
    dp_rank: int
    tp_rank: int
    pp_group: Optional[dist.ProcessGroup]
    dp_group: Optional[dist.ProcessGroup]
    tp_group: Optional[dist.ProcessGroup]


def init_mesh(pp_size: int = 1, dp_size: int = 1, tp_size: int = 1) -> ParallelMesh:
    """Creates the pp/dp/tp groups (collective: every rank must call it with the same sizes)."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    if pp_size * dp_size * tp_size != world:
        raise ValueError(f"pp {pp_size} x dp {dp_size} x tp {tp_size} != world size {world}")
    tp_rank = rank % tp_size
    pp_rank = (rank // tp_size) % pp_size
    dp_rank = rank // (tp_size * pp_size)
    pp_group = dp_group = tp_group = None
    if world > 1:
        for d in range(dp_size):
            for t in range(tp_size):
                ranks = [(d * pp_size + p) * tp_size + t for p in range(pp_size)]
                g = dist.new_group(ranks)
                if d == dp_rank and t == tp_rank:
                    pp_group = g
        for p in range(pp_size):
            for t in range(tp_size):
                ranks = [(d * pp_size + p) * tp_size + t for d in range(dp_size)]
                g = dist.new_group(ranks)
                if p == pp_rank and t == tp_rank:
                    dp_group = g
        for d in range(dp_size):
            for p in range(pp_size):
                ranks = [(d * pp_size + p) * tp_size + t for t in range(tp_size)]
                g = dist.new_group(ranks)
                if d == dp_rank and p == pp_rank:
                    tp_group = g
    return ParallelMesh(pp_size, dp_size, tp_size, pp_rank, dp_rank, tp_rank, pp_group, dp_group, tp_group)
