"""Convenience builders that assemble stages, schedule and optimizer for the model families of this package.

These are thin: everything they do can be done by hand with ``ManualPipelineStage`` (or ``pipeline()`` +
``PipelineStage``), a ``Schedule*`` class and ``FusedAdamW``; the benchmark and the examples use them so that they
exercise exactly the public API a user would.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, List, Optional

import torch
import torch.distributed as dist

from .manual_stage import ManualPipelineStage
from .models.llama import LlamaConfig, build_llama_stage, causal_lm_loss
from .optim import FlatParams, FusedAdamW
from .schedules import (
    Schedule1F1B,
    ScheduleGPipe,
    ScheduleInterleaved1F1B,
    ScheduleInterleavedZeroBubble,
    ScheduleZBVZeroBubble,
    ScheduleLoopedBFS,
)

SCHEDULES = {
    "gpipe": ScheduleGPipe,
    "1f1b": Schedule1F1B,
    "looped_bfs": ScheduleLoopedBFS,
    "interleaved_1f1b": ScheduleInterleaved1F1B,
    "zero_bubble": ScheduleInterleavedZeroBubble,
    "zbv": ScheduleZBVZeroBubble,  # V-shaped placement: rank r holds stages r and 2P-1-r
}


@dataclass
class Pipeline:
    stages: List[ManualPipelineStage]
    schedule: Any
    optimizer: Optional[FusedAdamW]
    flat: Optional[FlatParams]
    n_microbatches: int
    holds_first: bool
    holds_last: bool
    losses: List[torch.Tensor] = field(default_factory=list)

    tied: Any = None
    pre_optimizer: List[Callable[[], None]] = field(default_factory=list)  # run after the schedule, before the update

    def train_step(self, inputs=None, target=None) -> Optional[torch.Tensor]:
        """One optimizer step over one global batch. The rank holding the first stage passes ``inputs``, the rank
        holding the last stage passes ``target`` and gets the mean loss (a device scalar) back."""
        self.losses.clear()
        args = (inputs,) if self.holds_first and inputs is not None else ()
        if self.holds_last:
            self.schedule.step(*args, target=target, losses=self.losses)
        else:
            self.schedule.step(*args)
        if self.tied is not None:
            self.tied.sync_grads()
        for hook in self.pre_optimizer:
            hook()
        if self.optimizer is not None:
            self.optimizer.step(grad_scale=1.0 / self.n_microbatches, zero_grad=True)
        if self.holds_last and self.losses:
            return torch.stack([l.detach() for l in self.losses]).mean()
        return None


def build_llama_pipeline(
    cfg: LlamaConfig,
    global_batch: int,
    seq_len: int,
    n_microbatches: int,
    device: torch.device,
    schedule: str = "interleaved_1f1b",
    virtual_stages: int = 1,
    group: Optional[dist.ProcessGroup] = None,
    dtype: torch.dtype = torch.bfloat16,
    lr: float = 3e-4,
    weight_decay: float = 0.1,
    master_weights: bool = False,
    with_optimizer: bool = True,
    grad_reducer: Any = None,
    seed: int = 0,
    record_timing: bool = False,
    schedule_kwargs: Optional[dict] = None,
    balance: Any = True,
    dp_group: Optional[dist.ProcessGroup] = None,
    activation_checkpointing: bool = False,
) -> Pipeline:
    """Builds this rank's Llama stages (stage ``rank + k * pp_size`` for k < virtual_stages), the schedule and
    the fused optimizer."""
    if dist.is_initialized():
        pp_rank, pp_size = dist.get_rank(group), dist.get_world_size(group)
    else:
        pp_rank, pp_size = 0, 1
    num_stages = pp_size * virtual_stages
    if global_batch % n_microbatches != 0:
        raise ValueError(f"global batch {global_batch} is not divisible into {n_microbatches} microbatches")
    mb = global_batch // n_microbatches
    stages: List[ManualPipelineStage] = []
    params = []
    placement = None
    if schedule == "zbv":
        if virtual_stages != 2:
            raise ValueError("the V-shaped schedule runs exactly 2 stages per rank")
        from .schedules import v_placement

        placement = v_placement(pp_size)
    held = (sorted(s for s, r in placement.items() if r == pp_rank) if placement is not None
            else [pp_rank + k * pp_size for k in range(virtual_stages)])
    last_rank = placement[num_stages - 1] if placement is not None else (num_stages - 1) % pp_size
    for s in held:
        torch.manual_seed(seed + s)
        module = build_llama_stage(cfg, s, num_stages, device=device, dtype=dtype, pp_size=pp_size, seq_len=seq_len,
                                   balance=balance, stage_to_rank=placement,
                                   activation_checkpointing=activation_checkpointing)
        inp = (torch.empty(mb, seq_len, dtype=torch.int64, device="meta") if s == 0
               else torch.empty(mb, seq_len, cfg.dim, dtype=dtype, device="meta"))
        out = (torch.empty(mb, seq_len, cfg.vocab_size, dtype=dtype, device="meta") if s == num_stages - 1
               else torch.empty(mb, seq_len, cfg.dim, dtype=dtype, device="meta"))
        # a stage that starts or ends inside a layer's attention or MLP half also takes / hands over that half's
        # intermediate (the attention output or the SwiGLU output)
        if module.carry_in:
            inp = (inp, torch.empty(mb, seq_len, module.carry_in, dtype=dtype, device="meta"))
        if module.carry_out:
            out = (out, torch.empty(mb, seq_len, module.carry_out, dtype=dtype, device="meta"))
        stages.append(ManualPipelineStage(module, s, num_stages, device, n_microbatches, input_args=inp,
                                          output_args=out, group=group))
        params.extend(module.parameters())
    flat = opt = None
    if with_optimizer:
        flat = FlatParams(params)
        opt = FusedAdamW(flat, lr=lr, weight_decay=weight_decay, master_weights=master_weights)
        if dp_group is not None and grad_reducer is None:
            from .parallel.dp import GradReducer

            grad_reducer = GradReducer(flat, dp_group)
    cls = SCHEDULES[schedule]
    kw = dict(schedule_kwargs or {})
    kw.update(loss_fn=causal_lm_loss, grad_reducer=grad_reducer, record_timing=record_timing, return_outputs=False)
    if schedule in ("gpipe", "1f1b"):
        if virtual_stages != 1:
            raise ValueError(f"schedule {schedule!r} runs one stage per rank")
        sched = cls(stages[0], n_microbatches, **kw)
    else:
        sched = cls(stages, n_microbatches, **kw)
    return Pipeline(stages, sched, opt, flat, n_microbatches, holds_first=(pp_rank == 0),
                    holds_last=(last_rank == pp_rank))


def build_gpt2_pipeline(
    cfg,
    global_batch: int,
    seq_len: int,
    n_microbatches: int,
    device: torch.device,
    schedule: str = "1f1b",
    virtual_stages: int = 1,
    group: Optional[dist.ProcessGroup] = None,
    dp_group: Optional[dist.ProcessGroup] = None,
    dtype: torch.dtype = torch.bfloat16,
    lr: float = 3e-4,
    weight_decay: float = 0.1,
    seed: int = 0,
    record_timing: bool = False,
    balance: bool = False,
) -> Pipeline:
    """GPT-2 stages + schedule + fused optimizer for this rank; ``global_batch`` is the batch of ONE data-parallel
    replica. With ``dp_group`` the stage gradients are reduced by the fused NVLink all-reduce as each stage
    finishes its backward; the tied embedding / LM head is kept in sync across the first and last pipeline rank."""
    from .models.gpt2 import TiedEmbeddingSync, build_gpt2_stage, gpt2_loss

    if dist.is_initialized():
        pp_rank, pp_size = dist.get_rank(group), dist.get_world_size(group)
    else:
        pp_rank, pp_size = 0, 1
    num_stages = pp_size * virtual_stages
    mb = global_batch // n_microbatches
    stages: List[ManualPipelineStage] = []
    params = []
    placement = None
    if schedule == "zbv":
        # V shape: embedding and LM head share rank 0, so the tied weight needs no cross-rank synchronisation
        if virtual_stages != 2:
            raise ValueError("the V-shaped schedule runs exactly 2 stages per rank")
        from .schedules import v_placement

        placement = v_placement(pp_size)
    held = (sorted(s for s, r in placement.items() if r == pp_rank) if placement is not None
            else [pp_rank + k * pp_size for k in range(virtual_stages)])
    last_rank = placement[num_stages - 1] if placement is not None else (num_stages - 1) % pp_size
    for s in held:
        torch.manual_seed(seed + s)
        module = build_gpt2_stage(cfg, s, num_stages, device=device, dtype=dtype, balance=balance)
        inp = (torch.empty(mb, seq_len, dtype=torch.int64, device="meta") if s == 0
               else torch.empty(mb, seq_len, cfg.dim, dtype=dtype, device="meta"))
        out = (torch.empty(mb, seq_len, cfg.padded_vocab, dtype=dtype, device="meta") if s == num_stages - 1
               else torch.empty(mb, seq_len, cfg.dim, dtype=dtype, device="meta"))
        stages.append(ManualPipelineStage(module, s, num_stages, device, n_microbatches, input_args=inp,
                                          output_args=out, group=group))
        params.extend(module.parameters())
    first_local = next((st for st in stages if st.is_first), None)
    last_local = next((st for st in stages if st.is_last), None)
    if first_local is not None and last_local is not None and first_local is not last_local:
        # both ends of the pipeline on this rank: the head simply uses the embedding parameter
        last_local.submod.lm_head.weight = first_local.submod.wte.weight
    params = [p_ for st in stages for p_ in st.submod.parameters()]
    seen, unique = set(), []
    for p_ in params:
        if id(p_) not in seen:
            seen.add(id(p_))
            unique.append(p_)
    tied = TiedEmbeddingSync(stages, group, last_rank=last_rank)
    tied.broadcast()
    flat = FlatParams(unique)
    opt = FusedAdamW(flat, lr=lr, weight_decay=weight_decay)
    reducer = None
    if dp_group is not None:
        from .parallel.dp import GradReducer

        reducer = GradReducer(flat, dp_group)
    cls = SCHEDULES[schedule]
    kw = dict(loss_fn=gpt2_loss(cfg), grad_reducer=reducer, record_timing=record_timing, return_outputs=False)
    sched = cls(stages[0], n_microbatches, **kw) if schedule in ("gpipe", "1f1b") else cls(stages, n_microbatches, **kw)
    return Pipeline(stages, sched, opt, flat, n_microbatches, holds_first=(pp_rank == 0),
                    holds_last=(last_rank == pp_rank), tied=tied)


def build_mixtral_pipeline(
    cfg,
    global_batch: int,
    seq_len: int,
    n_microbatches: int,
    device: torch.device,
    schedule: str = "1f1b",
    virtual_stages: int = 1,
    pp_group: Optional[dist.ProcessGroup] = None,
    ep_group: Optional[dist.ProcessGroup] = None,
    dtype: torch.dtype = torch.bfloat16,
    lr: float = 3e-4,
    weight_decay: float = 0.1,
    seed: int = 0,
    record_timing: bool = False,
    capacity_factor: Optional[float] = None,
) -> Pipeline:
    """Mixtral stages for a PP x EP layout. ``global_batch`` is the batch of ONE expert-parallel rank (EP ranks are
    data-parallel replicas for the dense layers): dense gradients are averaged over ``ep_group`` with the fused
    all-reduce, expert gradients stay local, token rows travel through the fused dispatch/combine kernels."""
    from .models.mixtral import build_mixtral_stage
    from .parallel.ep import EPContext

    if dist.is_initialized():
        pp_rank, pp_size = dist.get_rank(pp_group), dist.get_world_size(pp_group)
        ep_rank = dist.get_rank(ep_group) if ep_group is not None else 0
        ep_size = dist.get_world_size(ep_group) if ep_group is not None else 1
    else:
        pp_rank, pp_size, ep_rank, ep_size = 0, 1, 0, 1
    num_stages = pp_size * virtual_stages
    mb = global_batch // n_microbatches
    ep = None
    if device.type == "cuda" and (ep_size > 1 or ep_group is not None or not dist.is_initialized()):
        ep = EPContext(ep_group, max_tokens=mb * seq_len, hidden=cfg.dim, top_k=cfg.top_k, n_experts=cfg.n_experts,
                       device=device,
                       # default: room for the worst case (every rank sends everything here), so no routing can
                       # overflow; only the rows in use are computed on, the rest is address space
                       capacity_factor=float(ep_size) if capacity_factor is None else capacity_factor)
    stages: List[ManualPipelineStage] = []
    dense, experts = [], []
    for k in range(virtual_stages):
        s = pp_rank + k * pp_size
        torch.manual_seed(seed + s)  # dense parameters start identical on every expert-parallel rank
        module = build_mixtral_stage(cfg, s, num_stages, ep, ep_size, ep_rank, device=device, dtype=dtype)
        inp = (torch.empty(mb, seq_len, dtype=torch.int64, device="meta") if s == 0
               else torch.empty(mb, seq_len, cfg.dim, dtype=dtype, device="meta"))
        out = (torch.empty(mb, seq_len, cfg.vocab_size, dtype=dtype, device="meta") if s == num_stages - 1
               else torch.empty(mb, seq_len, cfg.dim, dtype=dtype, device="meta"))
        stages.append(ManualPipelineStage(module, s, num_stages, device, n_microbatches, input_args=inp,
                                          output_args=out, group=pp_group))
        dense.extend(module.dense_parameters())
        experts.extend(module.expert_parameters())
    flat_dense = FlatParams(dense)
    groups = [flat_dense] + ([FlatParams(experts)] if experts else [])
    opt = FusedAdamW(groups, lr=lr, weight_decay=weight_decay)
    reducer = None
    if ep_size > 1:
        from .parallel.dp import GradReducer

        reducer = GradReducer(flat_dense, ep_group)
    cls = SCHEDULES[schedule]
    kw = dict(loss_fn=causal_lm_loss, grad_reducer=reducer, record_timing=record_timing, return_outputs=False)
    sched = cls(stages[0], n_microbatches, **kw) if schedule in ("gpipe", "1f1b") else cls(stages, n_microbatches, **kw)
    return Pipeline(stages, sched, opt, flat_dense, n_microbatches, holds_first=(pp_rank == 0),
                    holds_last=((num_stages - 1) % pp_size == pp_rank))


def build_llama_tp_pipeline(
    cfg: LlamaConfig,
    global_batch: int,
    seq_len: int,
    n_microbatches: int,
    device: torch.device,
    schedule: str = "1f1b",
    pp_group: Optional[dist.ProcessGroup] = None,
    tp_group: Optional[dist.ProcessGroup] = None,
    dtype: torch.dtype = torch.bfloat16,
    lr: float = 3e-4,
    weight_decay: float = 0.1,
    seed: int = 0,
    record_timing: bool = False,
) -> Pipeline:
    """Llama stages under tensor (+ sequence) x pipeline parallelism, one stage per pipeline rank.  Every
    tensor-parallel rank of the first stage receives the same token ids and every one of the last stage the same
    labels; between stages each rank ships its own token shard ``[mb * seq / tp, dim]`` to the same tensor-parallel
    rank of the next stage."""
    from .models.llama_tp import build_tp_llama_stage
    from .parallel.tp import TPContext

    if schedule not in ("gpipe", "1f1b"):
        raise ValueError("the tensor-parallel builder runs one stage per pipeline rank (gpipe or 1f1b)")
    pp_rank, pp_size = dist.get_rank(pp_group), dist.get_world_size(pp_group)
    tp_rank, tp_size = dist.get_rank(tp_group), dist.get_world_size(tp_group)
    mb = global_batch // n_microbatches
    rows = mb * seq_len // tp_size
    if device.type == "cuda":
        tp = TPContext(tp_group, max_rows=rows, max_cols=max(cfg.dim, 2 * cfg.ffn_dim // tp_size), device=device)
    else:
        # CPU (tests): the layers fall back to plain all-gather / reduce-scatter statements and only need the group
        from types import SimpleNamespace

        tp = SimpleNamespace(group=tp_group, world=tp_size, rank=tp_rank)
    torch.manual_seed(seed + pp_rank * 100 + tp_rank)
    module = build_tp_llama_stage(cfg, pp_rank, pp_size, tp, tp_size, tp_rank, mb, seq_len, device=device, dtype=dtype)
    first, last = pp_rank == 0, pp_rank == pp_size - 1
    inp = (torch.empty(mb, seq_len, dtype=torch.int64, device="meta") if first
           else torch.empty(rows, cfg.dim, dtype=dtype, device="meta"))
    out = (torch.empty(mb, seq_len, cfg.vocab_size, dtype=dtype, device="meta") if last
           else torch.empty(rows, cfg.dim, dtype=dtype, device="meta"))
    stage = ManualPipelineStage(module, pp_rank, pp_size, device, n_microbatches, input_args=inp, output_args=out,
                                group=pp_group)
    # Sharded weights have local gradients.  The LM head is replicated and sees all tokens on every rank, so its
    # gradient already agrees.  Norm weights and the embedding are replicated but work on this rank's token shard:
    # their gradients are partial sums and are added up over the tensor-parallel group (fused NVLink all-reduce).
    seq_parallel = [p_ for n, p_ in module.named_parameters()
                    if n.endswith("norm.weight") or n.startswith("tok_embeddings.")]
    ids_sp = {id(p_) for p_ in seq_parallel}
    rest = [p_ for p_ in module.parameters() if id(p_) not in ids_sp]
    if tp_size > 1:
        # replicated parameters start from tensor-parallel rank 0's values (the shards are seeded per rank)
        src = dist.get_global_rank(tp_group, 0) if tp_group is not None else 0
        for n, p_ in module.named_parameters():
            if id(p_) in ids_sp or n.startswith("output."):
                dist.broadcast(p_.data, src=src, group=tp_group)
    flat_sp, flat = FlatParams(seq_parallel), FlatParams(rest)
    opt = FusedAdamW([flat, flat_sp], lr=lr, weight_decay=weight_decay)
    hooks = []
    if tp_size > 1:
        from .parallel.dp import GradReducer

        reducer = GradReducer(flat_sp, tp_group, average=False)

        def _sum_sequence_parallel_grads():
            reducer.reduce_all()
            reducer.finish()

        hooks.append(_sum_sequence_parallel_grads)
    sched = SCHEDULES[schedule](stage, n_microbatches, loss_fn=causal_lm_loss, record_timing=record_timing,
                                return_outputs=False)
    return Pipeline([stage], sched, opt, flat, n_microbatches, holds_first=first, holds_last=last,
                    pre_optimizer=hooks)
