"""One communicator per directed pipeline link.

Every point-to-point transfer of the pipeline (activations downstream, gradients upstream) goes through a process
group that contains exactly the two ranks of that link and is used for that direction only.  On NCCL each such
group has its own communicator and stream, so a receive that was posted early and is still waiting for its sender
cannot hold up an unrelated send queued after it (with a single communicator all transfers of a rank share one
stream and block head-of-line).  The reference issues everything on the default group
(pippy/PipelineSchedule.py:200-222) and avoids the problem only by never posting a receive early.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Tuple

import torch.distributed as dist


def new_groups_worldwide(requests: List[List[int]], pg_options_factory=None) -> List[Optional[dist.ProcessGroup]]:
    """Creates process groups that only some ranks need, from inside code that runs on EVERY rank of the job.

    ``dist.new_group`` must be called by all ranks of the default group in the same order, members or not.  Each
    rank passes the global-rank lists it wants (a list may repeat: the k-th repeat is a distinct group); the
    requests are all-gathered, their union is put in one canonical order, and every rank creates every group.
    Returns the groups for this rank's own requests, in request order."""
    world = dist.get_world_size()
    keyed = []
    seen: Dict[Tuple[int, ...], int] = {}
    for ranks in requests:
        t = tuple(sorted(int(r) for r in ranks))
        k = seen.get(t, 0)
        seen[t] = k + 1
        keyed.append((t, k))
    gathered: List[Optional[list]] = [None] * world
    dist.all_gather_object(gathered, keyed)
    union = sorted({(tuple(a), int(b)) for g in gathered for a, b in g})
    made: Dict[tuple, Optional[dist.ProcessGroup]] = {}
    for ranks, k in union:
        opts = pg_options_factory() if pg_options_factory is not None else None
        made[(ranks, k)] = dist.new_group(list(ranks), pg_options=opts) if opts is not None else dist.new_group(list(ranks))
    return [made[key] for key in keyed]


class LinkGroups:
    """``groups[(src_group_rank, dst_group_rank, kind)]`` -> ProcessGroup, kind in {"F", "B"}."""

    def __init__(self, pp_group: Optional[dist.ProcessGroup], links: Iterable[Tuple[int, int]],
                 max_ctas: Optional[int] = None):
        """``max_ctas`` (default 2, or the environment variable ``PIPPY_P2P_MAX_CTAS``) caps the thread blocks of
        each link's NCCL kernels.  A point-to-point kernel spins on its
        SMs until the peer arrives; with the default channel count it would take dozens of SMs away from the
        persistent compute kernels for that long.  Two blocks move a 64 MiB activation in about a millisecond,
        which hides behind tens of milliseconds of stage compute."""
        import os

        if max_ctas is None:
            max_ctas = int(os.environ.get("PIPPY_P2P_MAX_CTAS", "2"))
        self.pp_group = pp_group
        self.groups: Dict[Tuple[int, int, str], dist.ProcessGroup] = {}
        if not dist.is_initialized():
            return
        world = dist.get_world_size(pp_group)
        seen = set()
        ordered: List[Tuple[int, int]] = []
        for a, b in sorted(set((int(a), int(b)) for a, b in links)):
            if a == b or (a, b) in seen:
                continue
            seen.add((a, b))
            ordered.append((a, b))
        def make_options():
            if dist.get_backend(pp_group) != "nccl":
                return None
            try:
                opts = dist.ProcessGroupNCCL.Options()
                opts.is_high_priority_stream = True
                opts.config.max_ctas = max_ctas
                opts.config.min_ctas = 1
                return opts
            except Exception:  # pragma: no cover - older bindings without per-communicator config
                return None

        me = dist.get_rank(pp_group)
        requests, keys = [], []
        for a, b in ordered:
            if me not in (a, b):
                continue
            ranks = sorted({a, b})
            global_ranks = [dist.get_global_rank(pp_group, r) if pp_group is not None else r for r in ranks]
            requests += [global_ranks, global_ranks]  # one communicator per direction
            keys += [(a, b, "F"), (b, a, "B")]
        groups = new_groups_worldwide(requests, make_options if dist.get_backend(pp_group) == "nccl" else None)
        for key, g in zip(keys, groups):
            self.groups[key] = g

    def get(self, src: int, dst: int, kind: str) -> Optional[dist.ProcessGroup]:
        return self.groups.get((src, dst, kind))


def pipeline_links(num_stages: int, pp_size: int, dests: Optional[Dict[int, List[int]]] = None,
                   stage_to_rank: Optional[Dict[int, int]] = None) -> List[Tuple[int, int]]:
    """Directed rank pairs (producer rank, consumer rank) of a pipeline; stage s lives on rank
    ``stage_to_rank[s]``, by default s % pp_size."""
    out = []
    if dests is None:
        dests = {s: ([s + 1] if s + 1 < num_stages else []) for s in range(num_stages)}
    where = (lambda s: stage_to_rank[s]) if stage_to_rank is not None else (lambda s: s % pp_size)
    for s, ds in dests.items():
        for d in ds:
            a, b = where(s), where(d)
            if a != b and (a, b) not in out:
                out.append((a, b))
    return out
