"""Reference arms of the composed benchmark configs: the pipeline runtime the reference migrated into
(``torch.distributed.pipelining``) composed with the stock PyTorch library for the second dimension, the way the
reference's own tests and examples compose them:

* ``gpt2-pp4dp2``      PipelineStage + Schedule1F1B over ``DistributedDataParallel`` stage modules
                       (test/test_composability.py:203-300 wraps stage modules in DDP the same way).
* ``llama13b-tp4pp2``  DTensor tensor / sequence parallelism (``parallelize_module`` with Colwise / Rowwise /
                       SequenceParallel styles) inside each stage, PipelineStage + Schedule1F1B across them
                       (examples/tp+pp/pippy_tp.py:79-153 builds the same 2-D mesh).
* ``mixtral-pp2ep4``   experts sharded over the expert-parallel group, tokens exchanged with the differentiable
                       ``all_to_all_single`` and a loop over local experts (examples/mixture_of_experts/dist_moe.py:43-59),
                       dense layers under DDP over the same group, PipelineStage + Schedule1F1B across stages.

Models are plain eager PyTorch (nn.Linear, nn.LayerNorm / nn.RMSNorm, F.scaled_dot_product_attention,
F.cross_entropy); nothing from pippy_b200 is imported.  ``PIPPY_REF_DEVICE=cpu`` runs the same code on gloo in
fp32 so that the arms can be exercised without GPUs (small ``--layers / --seq / --batch``).
"""
import json
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def _rope_tables(hd, theta, seq_len, dtype, device):
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32, device=device) / hd))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32, device=device), inv)
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(dtype)[None, None], emb.sin().to(dtype)[None, None]


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2 :]
    return torch.cat((-x2, x1), dim=-1)


def _init(module, std=0.02):
    for m in module.modules():
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=std)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)


# ----------------------------------------------------------------------------------------------------- GPT-2

class GPT2Block(nn.Module):
    def __init__(self, d, heads, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.d, self.heads = d, heads
        self.ln_1 = nn.LayerNorm(d, eps=1e-5, **kw)
        self.c_attn = nn.Linear(d, 3 * d, **kw)
        self.c_proj = nn.Linear(d, d, **kw)
        self.ln_2 = nn.LayerNorm(d, eps=1e-5, **kw)
        self.c_fc = nn.Linear(d, 4 * d, **kw)
        self.mlp_proj = nn.Linear(4 * d, d, **kw)

    def forward(self, x):
        B, S, d = x.shape
        q, k, v = (t.view(B, S, self.heads, d // self.heads).transpose(1, 2)
                   for t in self.c_attn(self.ln_1(x)).split(d, dim=2))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.c_proj(a.transpose(1, 2).reshape(B, S, d))
        return x + self.mlp_proj(F.gelu(self.c_fc(self.ln_2(x)), approximate="tanh"))


class GPT2Stage(nn.Module):
    """A contiguous slice of GPT-2.  The LM head has its own weight: the reference has no tied-parameter
    synchronisation for training, so a stock pipeline leaves the head untied when it sits on another rank."""

    def __init__(self, layer_ids, first, last, vocab, n_pos, d, heads, dtype, device):
        super().__init__()
        self.first, self.last = first, last
        kw = dict(dtype=dtype, device=device)
        if first:
            self.wte = nn.Embedding(vocab, d, **kw)
            self.wpe = nn.Embedding(n_pos, d, **kw)
        self.h = nn.ModuleDict({str(i): GPT2Block(d, heads, dtype, device) for i in layer_ids})
        if last:
            self.ln_f = nn.LayerNorm(d, eps=1e-5, **kw)
            self.lm_head = nn.Linear(d, vocab, bias=False, **kw)
        _init(self)

    def forward(self, x):
        if self.first:
            pos = torch.arange(x.shape[1], device=x.device)
            x = self.wte(x) + self.wpe(pos)[None]
        for blk in self.h.values():
            x = blk(x)
        if self.last:
            x = self.lm_head(self.ln_f(x))
        return x


# --------------------------------------------------------------------------- Llama block shared by TP and MoE

class Attention(nn.Module):
    def __init__(self, d, n_heads, kv_heads, dtype, device):
        super().__init__()
        kw = dict(bias=False, dtype=dtype, device=device)
        self.hd = d // n_heads
        self.groups = n_heads // kv_heads
        self.q_proj = nn.Linear(d, n_heads * self.hd, **kw)
        self.k_proj = nn.Linear(d, kv_heads * self.hd, **kw)
        self.v_proj = nn.Linear(d, kv_heads * self.hd, **kw)
        self.o_proj = nn.Linear(n_heads * self.hd, d, **kw)

    def forward(self, h, cos, sin):
        B, S, _ = h.shape
        # -1 heads: under tensor parallelism each rank's projections hold its share of the heads
        q = self.q_proj(h).view(B, S, -1, self.hd).transpose(1, 2)
        k = self.k_proj(h).view(B, S, -1, self.hd).transpose(1, 2)
        v = self.v_proj(h).view(B, S, -1, self.hd).transpose(1, 2)
        q = q * cos + _rotate_half(q) * sin
        k = k * cos + _rotate_half(k) * sin
        if self.groups > 1:
            k = k.repeat_interleave(self.groups, dim=1)
            v = v.repeat_interleave(self.groups, dim=1)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.o_proj(a.transpose(1, 2).reshape(B, S, -1))


class SwiGLU(nn.Module):
    def __init__(self, d, ffn, dtype, device):
        super().__init__()
        kw = dict(bias=False, dtype=dtype, device=device)
        self.gate_proj = nn.Linear(d, ffn, **kw)
        self.up_proj = nn.Linear(d, ffn, **kw)
        self.down_proj = nn.Linear(ffn, d, **kw)

    def forward(self, h):
        return self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class AllToAllMoE(nn.Module):
    """Top-k routed experts, ``n_experts / ep`` of them on each rank of ``group``: sort the (token, choice) rows by
    expert, exchange row counts, ``all_to_all_single`` the rows to the experts' ranks, run the local experts one
    after the other, ``all_to_all_single`` the results back and add them up weighted by the gate."""

    def __init__(self, d, ffn, n_experts, top_k, group, dtype, device):
        super().__init__()
        self.group = group
        self.ep = dist.get_world_size(group) if group is not None else 1
        self.E, self.k = n_experts, top_k
        self.epr = n_experts // self.ep
        self.gate = nn.Linear(d, n_experts, bias=False, dtype=dtype, device=device)
        self.experts = nn.ModuleList(SwiGLU(d, ffn, dtype, device) for _ in range(self.epr))

    def forward(self, x):
        from torch.distributed.nn.functional import all_to_all_single

        shape = x.shape
        x = x.reshape(-1, shape[-1])
        probs = F.softmax(self.gate(x).float(), dim=-1)
        topv, topi = probs.topk(self.k, dim=-1)
        topv = (topv / topv.sum(-1, keepdim=True)).to(x.dtype)
        flat_e = topi.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        tok = order // self.k
        rows = x[tok]
        counts = torch.bincount(flat_e, minlength=self.E)
        if self.ep > 1:
            counts_in = torch.empty_like(counts)
            dist.all_to_all_single(counts_in, counts, group=self.group)
            send = counts.view(self.ep, self.epr).sum(1).tolist()
            recv = counts_in.view(self.ep, self.epr).sum(1).tolist()
            got = all_to_all_single(rows.new_empty(sum(recv), rows.shape[1]), rows, recv, send, group=self.group)
        else:
            counts_in, got = counts, rows
        # rows arrive ordered by source rank, then by local expert
        expert_of_row = torch.repeat_interleave(
            torch.arange(self.epr, device=x.device).repeat(self.ep), counts_in.reshape(-1))
        out = torch.zeros_like(got)
        for e, expert in enumerate(self.experts):
            idx = (expert_of_row == e).nonzero(as_tuple=True)[0]
            if idx.numel():
                out = out.index_add(0, idx, expert(got[idx]))
        if self.ep > 1:
            out = all_to_all_single(rows.new_empty(sum(send), rows.shape[1]), out, send, recv, group=self.group)
        y = torch.zeros_like(x).index_add(0, tok, out * topv.reshape(-1)[order][:, None])
        return y.view(shape)


class DecoderBlock(nn.Module):
    def __init__(self, d, n_heads, kv_heads, eps, mlp, dtype, device):
        super().__init__()
        self.input_layernorm = nn.RMSNorm(d, eps=eps, dtype=dtype, device=device)
        self.attn = Attention(d, n_heads, kv_heads, dtype, device)
        self.post_attention_layernorm = nn.RMSNorm(d, eps=eps, dtype=dtype, device=device)
        self.mlp = mlp

    def forward(self, x, cos, sin):
        x = x + self.attn(self.input_layernorm(x), cos, sin)
        return x + self.mlp(self.post_attention_layernorm(x))


class DecoderStage(nn.Module):
    def __init__(self, blocks, first, last, vocab, d, hd, eps, theta, seq_len, dtype, device):
        super().__init__()
        self.first, self.last = first, last
        if first:
            self.embed_tokens = nn.Embedding(vocab, d, dtype=dtype, device=device)
        self.layers = nn.ModuleDict(blocks)
        if last:
            self.norm = nn.RMSNorm(d, eps=eps, dtype=dtype, device=device)
            self.lm_head = nn.Linear(d, vocab, bias=False, dtype=dtype, device=device)
        cos, sin = _rope_tables(hd, theta, seq_len, dtype, device)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)
        _init(self)

    def forward(self, x):
        if self.first:
            x = self.embed_tokens(x)
        for blk in self.layers.values():
            x = blk(x, self.cos, self.sin)
        if self.last:
            x = self.lm_head(self.norm(x))
        return x


def _tensor_parallel(stage: DecoderStage, tp_mesh) -> None:
    """Megatron-style sharding with sequence-parallel activations, in DTensor's parallel styles: between the
    parallel regions the residual stream is this rank's slice of the sequence."""
    from torch.distributed.tensor import Replicate, Shard
    from torch.distributed.tensor.parallel import (ColwiseParallel, PrepareModuleInput, RowwiseParallel,
                                                   SequenceParallel, parallelize_module)

    plan = {}
    if stage.first:
        plan["embed_tokens"] = RowwiseParallel(input_layouts=Replicate(), output_layouts=Shard(1))
    for name in stage.layers:
        p = f"layers.{name}."
        plan[p + "input_layernorm"] = SequenceParallel()
        plan[p + "attn"] = PrepareModuleInput(input_layouts=(Shard(1), None, None),
                                              desired_input_layouts=(Replicate(), None, None))
        for w in ("q_proj", "k_proj", "v_proj"):
            plan[p + "attn." + w] = ColwiseParallel()
        plan[p + "attn.o_proj"] = RowwiseParallel(output_layouts=Shard(1))
        plan[p + "post_attention_layernorm"] = SequenceParallel()
        plan[p + "mlp"] = PrepareModuleInput(input_layouts=(Shard(1),), desired_input_layouts=(Replicate(),))
        plan[p + "mlp.gate_proj"] = ColwiseParallel()
        plan[p + "mlp.up_proj"] = ColwiseParallel()
        plan[p + "mlp.down_proj"] = RowwiseParallel(output_layouts=Shard(1))
    if stage.last:
        plan["norm"] = SequenceParallel()
        plan["lm_head"] = ColwiseParallel(input_layouts=Shard(1), output_layouts=Replicate())
    parallelize_module(stage, tp_mesh, plan)


# ------------------------------------------------------------------------------------------------ job set-up

def _even_layers(n_layers, stage, num_stages):
    base, rem = divmod(n_layers, num_stages)
    start = stage * base + min(stage, rem)
    return range(start, start + base + (1 if stage < rem else 0))


def build_job(args, world, rank, device, dtype):
    """This rank's stage module, schedule and data slice for ``args.config``."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.pipelining import PipelineStage, Schedule1F1B, ScheduleGPipe
    from torch.nn.parallel import DistributedDataParallel as DDP

    inner_default = {"gpt2-pp4dp2": 2, "llama13b-tp4pp2": 4, "mixtral-pp2ep4": 4}[args.config]
    inner = getattr(args, "inner", None) or (inner_default if world % inner_default == 0 else 2)
    if world % inner:
        raise ValueError(f"{args.config} needs a multiple of {inner} ranks, got {world}")
    pp = world // inner
    second = {"gpt2-pp4dp2": "dp", "llama13b-tp4pp2": "tp", "mixtral-pp2ep4": "ep"}[args.config]
    mesh = init_device_mesh(device.type, (pp, inner), mesh_dim_names=("pp", second))
    pp_rank, in_rank = mesh.get_local_rank("pp"), mesh.get_local_rank(second)
    pp_group, in_group = mesh["pp"].get_group(), mesh[second].get_group()
    first, last = pp_rank == 0, pp_rank == pp - 1
    n_mb, seq = args.microbatches, args.seq
    ddp_kw = dict(device_ids=[device.index]) if device.type == "cuda" else {}
    after_backward = None
    torch.manual_seed(1000 + pp_rank)  # replicas of a stage start from the same weights

    if args.config == "gpt2-pp4dp2":
        vocab, n_pos, d, n_layers, heads = 50257, 1024, 768, 12, 12
        n_layers = getattr(args, "layers", None) or n_layers
        if os.environ.get("PIPPY_REF_TINY"):
            vocab, d, heads = 512, 128, 2
        mod = GPT2Stage(_even_layers(n_layers, pp_rank, pp), first, last, vocab, max(n_pos, seq), d, heads, dtype, device)
        module = DDP(mod, process_group=in_group, **ddp_kw) if inner > 1 else mod
        replicas, replica = inner, in_rank
        rows, hidden = args.batch // inner // n_mb, (seq, d)
        desc = f"GPT-2 small ({n_layers}L, d{d}, vocab {vocab}, LM head untied)"
        parallelism = f"pp{pp}xdp{inner} (DistributedDataParallel stage modules)"
    elif args.config == "llama13b-tp4pp2":
        vocab, d, n_layers, heads, ffn = 32000, 5120, 40, 40, 13824
        if getattr(args, "layers", None):
            n_layers = args.layers
        if os.environ.get("PIPPY_REF_TINY"):
            vocab, d, heads, ffn = 512, 256, 4, 512
        blocks = {str(i): DecoderBlock(d, heads, heads, 1e-5, SwiGLU(d, ffn, dtype, device), dtype, device)
                  for i in _even_layers(n_layers, pp_rank, pp)}
        mod = DecoderStage(blocks, first, last, vocab, d, d // heads, 1e-5, 10000.0, seq, dtype, device)
        if inner > 1:
            # every tensor-parallel rank built the same full weights (same seed); DTensor keeps this rank's shard
            _tensor_parallel(mod, mesh[second])
        module = mod
        replicas, replica = 1, 0
        rows, hidden = args.batch // n_mb, (seq // inner, d)
        desc = f"Llama-2-13B shape ({n_layers}L, d{d}, {heads}h, ffn {ffn}, vocab {vocab})"
        parallelism = f"tp{inner}xpp{pp} (DTensor Colwise/Rowwise/SequenceParallel)"
    else:
        vocab, d, n_layers, heads, kv, ffn, E, k = 32000, 4096, 16, 32, 8, 14336, 8, 2
        if getattr(args, "layers", None):
            n_layers = args.layers
        if os.environ.get("PIPPY_REF_TINY"):
            vocab, d, heads, kv, ffn = 512, 256, 4, 2, 512
        blocks = {str(i): DecoderBlock(d, heads, kv, 1e-5,
                                       AllToAllMoE(d, ffn, E, k, in_group if inner > 1 else None, dtype, device),
                                       dtype, device)
                  for i in _even_layers(n_layers, pp_rank, pp)}
        mod = DecoderStage(blocks, first, last, vocab, d, d // heads, 1e-5, 1e6, seq, dtype, device)
        expert_params = [p for n, p in mod.named_parameters() if ".mlp.experts." in n]
        if inner > 1:
            # experts differ between ranks: re-draw them with a rank-specific seed, keep them out of DDP
            torch.manual_seed(5000 + rank)
            with torch.no_grad():
                for p in expert_params:
                    nn.init.normal_(p, std=0.02)
            DDP._set_params_and_buffers_to_ignore_for_model(
                mod, [n for n, _ in mod.named_parameters() if ".mlp.experts." in n])
            module = DDP(mod, process_group=in_group, **ddp_kw)

            def after_backward():
                # an expert sums the gradients of rows from every rank, each normalised by its own rank's token
                # count; 1 / ep puts them on the scale of the averaged dense gradients
                grads = [p.grad for p in expert_params if p.grad is not None]
                if grads:
                    torch._foreach_mul_(grads, 1.0 / inner)
        else:
            module = mod
        replicas, replica = inner, in_rank
        rows, hidden = args.batch // inner // n_mb, (seq, d)
        desc = f"Mixtral shape ({n_layers}L, d{d}, {heads}q/{kv}kv heads, {E} experts of ffn {ffn}, top-{k}; no aux loss)"
        parallelism = f"pp{pp}xep{inner} (all_to_all_single dispatch, DDP over the dense layers)"

    if rows < 1:
        raise ValueError("batch too small for this many microbatches and replicas")
    inp = (torch.empty(rows, seq, dtype=torch.int64, device="meta") if first
           else torch.empty(rows, *hidden, dtype=dtype, device="meta"))
    out = (torch.empty(rows, seq, vocab, dtype=dtype, device="meta") if last
           else torch.empty(rows, *hidden, dtype=dtype, device="meta"))
    stage = PipelineStage(module, pp_rank, pp, device, input_args=(inp,), output_args=(out,), group=pp_group)

    def loss_fn(logits, target):
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), target.reshape(-1), ignore_index=-100) / n_mb

    sched_cls, sched_name = (Schedule1F1B, "1f1b") if pp > 1 else (ScheduleGPipe, "gpipe")
    sched = sched_cls(stage, n_mb, loss_fn=loss_fn, scale_grads=False)
    return dict(sched=sched, params=list(mod.parameters()), first=first, last=last, replica=replica,
                replicas=replicas, vocab=vocab, desc=desc, parallelism=parallelism, schedule=sched_name,
                after_backward=after_backward, prints=(rank == 0))


def run(args, watchdog_cls, unavailable) -> None:
    import warnings

    warnings.filterwarnings("ignore")
    cpu = os.environ.get("PIPPY_REF_DEVICE", "") == "cpu"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        unavailable(f"{args.config} composes parallel dimensions: it needs 2 or more ranks")
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    if cpu:
        device, dtype = torch.device("cpu"), torch.float32
        dist.init_process_group("gloo")
    else:
        device, dtype = torch.device("cuda", local_rank), torch.bfloat16
        torch.cuda.set_device(device)
        dist.init_process_group("nccl", device_id=device)

    job = build_job(args, world, rank, device, dtype)
    sched, first, last = job["sched"], job["first"], job["last"]
    opt = torch.optim.AdamW(job["params"], lr=3e-4, weight_decay=0.1, fused=True)

    per = args.batch // job["replicas"]
    lo = job["replica"] * per
    g = torch.Generator().manual_seed(1234)
    host_ids, host_lbl = [], []
    for _ in range(2):
        ids = torch.randint(0, job["vocab"], (args.batch, args.seq), generator=g)[lo : lo + per].contiguous()
        lbl = torch.roll(ids, -1, dims=1)
        lbl[:, -1] = -100
        host_ids.append(ids if cpu else ids.pin_memory())
        host_lbl.append(lbl if cpu else lbl.pin_memory())
    dev_ids = [t.to(device) for t in host_ids]
    dev_lbl = [t.to(device) for t in host_lbl]

    def step(ids, lbl):
        losses = []
        if first and last:
            sched.step(ids, target=lbl, losses=losses)
        elif first:
            sched.step(ids)
        elif last:
            sched.step(target=lbl, losses=losses)
        else:
            sched.step()
        if job["after_backward"] is not None:
            job["after_backward"]()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return torch.stack(losses).sum() if losses else None

    def sync():
        if not cpu:
            torch.cuda.synchronize()

    def barrier():
        dist.barrier()
        sync()

    def reduce(x, op):
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=op)
        return float(t.item())

    class Span:
        """Device time between ``begin`` and ``end`` in ms (host clock on the CPU path)."""

        def begin(self):
            if cpu:
                self.t0 = time.perf_counter()
            else:
                self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                self.e0.record()

        def end(self):
            if cpu:
                self.t1 = time.perf_counter()
            else:
                self.e1.record()

        def ms(self):
            return (self.t1 - self.t0) * 1e3 if cpu else self.e0.elapsed_time(self.e1)

    dog = None
    if not cpu:
        dog = watchdog_cls(300.0, device)
        dog.start()

    def mark(what):
        if dog is not None:
            dog.mark(what)

    loss = None
    for i in range(args.warmup):
        t0 = time.time()
        loss = step(dev_ids[i % 2], dev_lbl[i % 2])
        mark(f"warm-up step {i + 1}")
        sync()
        if dog is not None and (i > 0 or args.warmup == 1):
            dog.set_step_time(time.time() - t0)
    barrier()
    mark("warm-up")
    sampler = None
    if not cpu and rank == 0:
        sys.path.insert(0, os.path.dirname(HERE))
        from bench import ClockSampler  # nvidia-smi sampling only; no model or engine code

        sampler = ClockSampler(local_rank)
        sampler.start()
    barrier()
    span = Span()
    span.begin()
    for i in range(args.steps):
        loss = step(dev_ids[i % 2], dev_lbl[i % 2])
        mark(f"timed step {i + 1}")
    span.end()
    barrier()
    ms_total = reduce(span.ms(), dist.ReduceOp.MAX)
    clocks = sampler.stop() if sampler is not None else None
    final_loss = reduce(float(loss.item()) if loss is not None else float("-inf"), dist.ReduceOp.MAX)

    e2e = None
    if not getattr(args, "no_e2e", False):
        h2d = d2h = 0
        barrier()
        span = Span()
        span.begin()
        for i in range(args.steps):
            ids = lbl = None
            if first:
                ids = host_ids[i % 2].to(device, non_blocking=True)
                h2d += ids.numel() * ids.element_size()
            if last:
                lbl = host_lbl[i % 2].to(device, non_blocking=True)
                h2d += lbl.numel() * lbl.element_size()
            l = step(ids, lbl)
            if l is not None:
                hl = l.float().cpu()
                d2h += hl.numel() * hl.element_size()
            mark(f"end-to-end step {i + 1}")
        span.end()
        barrier()
        e2e_ms = reduce(span.ms(), dist.ReduceOp.MAX)
        e2e = {
            "value": args.batch * args.seq * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s",
            "h2d_bytes_per_step": int(reduce(float(h2d), dist.ReduceOp.SUM) / args.steps),
            "d2h_bytes_per_step": int(reduce(float(d2h), dist.ReduceOp.SUM) / args.steps),
            "ms_per_step": e2e_ms / args.steps,
        }
    if dog is not None:
        dog.stop()
    if job["prints"]:
        print(json.dumps({
            "metric": "tokens/sec (whole job, device-timed, max over ranks)",
            "value": args.batch * args.seq * args.steps / (ms_total * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp32 (CPU exercise of the arm)" if cpu else "bf16",
            "data": "synthetic (uniform token ids, labels shifted by one; random-init weights)", "impl": "reference",
            "reference_system": "torch.distributed.pipelining",
            "config": {"name": args.config, "model": job["desc"], "global_batch": args.batch, "seq_len": args.seq,
                       "microbatches": args.microbatches, "parallelism": job["parallelism"],
                       "schedule": job["schedule"], "optimizer": "torch.optim.AdamW(fused=True) lr 3e-4",
                       "l2": "inputs larger than L2 (weights and activations stream every step)"},
            "final_loss": final_loss, "clocks": clocks, "e2e": e2e, "gpu_launches": 0,
        }), flush=True)
    dist.destroy_process_group()
