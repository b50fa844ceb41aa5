"""Gradient synchronisation of parameters that the splitter replicated across stages (tied weights).

``Pipe.replicated_params`` lists, per shared tensor, which stage holds a copy under which name.  Before the
optimizer step the copies' gradients must be summed so that all copies take the same update (the recipe the
reference's model tests spell out by hand, test/hf_test.py:1047-1062).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


def _grad_of(p: torch.nn.Parameter) -> Optional[torch.Tensor]:
    """The gradient to reduce.  A parameter that lives in a flat buffer has ``main_grad``; ops outside this
    package's kernels (and every op on the CPU path) still leave their share in ``.grad``, so that is folded into
    ``main_grad`` first: otherwise the reduction would sum zeros and the copies would drift apart."""
    mg = getattr(p, "main_grad", None)
    if mg is None:
        return p.grad
    if p.grad is not None:
        mg.add_(p.grad.to(mg.dtype))
        p.grad = None
    return mg


def _get(module, qualname: str):
    obj = module
    for atom in qualname.split("."):
        obj = getattr(obj, atom)
    return obj


class TiedParamSync:
    """Created once on every pipeline rank (process groups are made collectively); call :meth:`sync` after the
    schedule's step and before the optimizer's."""

    def __init__(self, pipe, local_stages: Sequence, pp_group: Optional[dist.ProcessGroup] = None):
        self.entries = []
        world = dist.get_world_size(pp_group) if dist.is_initialized() else 1
        rank = dist.get_rank(pp_group) if dist.is_initialized() else 0
        by_index = {s.stage_index: s for s in local_stages}
        from ..comm.p2p import new_groups_worldwide

        wanted, pending = [], []
        for group in pipe.replicated_params:
            stage_ids = sorted(int(name.split("_")[-1]) for name in group)
            where = (local_stages[0].rank_of_stage if local_stages else (lambda sid: sid % world))
            ranks = sorted({where(sid) for sid in stage_ids})
            local = [(by_index[sid], group[f"submod_{sid}"]) for sid in stage_ids if sid in by_index]
            need = len(ranks) > 1 and rank in ranks
            if need:
                wanted.append([dist.get_global_rank(pp_group, r) if pp_group is not None else r for r in ranks])
            pending.append((ranks, need, local))
        made = iter(new_groups_worldwide(wanted)) if dist.is_initialized() else iter(())
        for ranks, need, local in pending:
            self.entries.append((ranks, next(made) if need else None, local, rank in ranks))

    @torch.no_grad()
    def sync(self) -> None:
        for ranks, pg, local, member in self.entries:
            if not member or not local:
                continue
            params = [_get(stage.submod, qual) for stage, qual in local]
            grads = [_grad_of(p) for p in params]
            total = None
            for g in grads:
                if g is not None:
                    total = g.clone() if total is None else total + g
            if total is None:
                total = torch.zeros_like(params[0], dtype=torch.float32 if hasattr(params[0], "main_grad") else params[0].dtype)
            if pg is not None:
                dist.all_reduce(total, group=pg)
            for p in params:
                if getattr(p, "main_grad", None) is not None:
                    p.main_grad.copy_(total)
                else:
                    p.grad = total.clone().to(p.dtype)
