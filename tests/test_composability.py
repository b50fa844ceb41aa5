"""Pipeline x data parallel composition on a 2 x 2 gloo mesh: GPT-2 stages with a tied embedding / LM head, stage
gradients reduced at the schedule's REDUCE_GRAD action (reference test/test_composability.py: grads equal the
single-process grads averaged over the replicas)."""
import pytest
import torch

from _mp import run_ranks


def _pp_dp(rank, world, schedule, scale_grads=False):
    import torch.distributed as dist

    from pippy_b200.models.gpt2 import GPT2Config
    from pippy_b200.parallel.mesh import init_mesh
    from pippy_b200.train import build_gpt2_pipeline

    mesh = init_mesh(pp_size=2, dp_size=2)
    assert dist.get_world_size(mesh.pp_group) == 2 and dist.get_world_size(mesh.dp_group) == 2
    cfg = GPT2Config.tiny()
    B, S, n_mb = 4, 16, 2
    v = 1 if schedule == "1f1b" else 2
    pipe = build_gpt2_pipeline(cfg, B, S, n_mb, torch.device("cpu"), schedule=schedule, virtual_stages=v,
                               group=mesh.pp_group, dp_group=mesh.dp_group, dtype=torch.float32, lr=0.0, weight_decay=0.0)
    # with both a reducer and scale_grads the scaling must come after the reduction has been waited for
    pipe.schedule.scale_grads = scale_grads
    gen = torch.Generator().manual_seed(100)
    data = [torch.randint(0, cfg.vocab_size, (B, S), generator=gen) for _ in range(2)]  # one batch per replica
    ids = data[mesh.dp_rank]

    # run the schedule but stop before the optimizer: compare the reduced gradients
    pipe.losses.clear()
    if pipe.holds_first and pipe.holds_last:
        pipe.schedule.step(ids, target=ids, losses=pipe.losses)
    elif pipe.holds_first:
        pipe.schedule.step(ids)
    elif pipe.holds_last:
        pipe.schedule.step(target=ids, losses=pipe.losses)
    else:
        pipe.schedule.step()
    pipe.tied.sync_grads()
    pipe.flat.fold_autograd_grads()

    # oracle: every stage rebuilt locally with the same seeds, run on both replicas' batches, gradients averaged
    total = {}
    for d in range(2):
        from pippy_b200.models.gpt2 import build_gpt2_stage, gpt2_loss

        n_stages = pipe.stages[0].num_stages
        full = []
        for s in range(n_stages):
            torch.manual_seed(0 + s)
            full.append(build_gpt2_stage(cfg, s, n_stages, dtype=torch.float32))
        full[-1].lm_head.weight = full[0].wte.weight  # tied
        loss_fn = gpt2_loss(cfg)
        for mb_ids in torch.tensor_split(data[d], n_mb):
            h = mb_ids
            for m in full:
                h = m(h)
            loss_fn(h, mb_ids).backward()
        for s, m in enumerate(full):
            for k, p in m.named_parameters():
                if p.grad is not None:
                    total[(s, k)] = total.get((s, k), 0) + p.grad / 2
    for st in pipe.stages:
        for k, p in st.submod.named_parameters():
            want = total.get((st.stage_index, k))
            if want is None and k == "lm_head.weight":
                want = total[(0, "wte.weight")]
            if scale_grads:
                want = want / n_mb
            torch.testing.assert_close(p.main_grad, want, rtol=2e-4, atol=2e-5, msg=f"{schedule} stage {st.stage_index} {k}")
    dist.barrier()


@pytest.mark.parametrize("schedule", ["1f1b", "zero_bubble"])
def test_pp2_dp2_gpt2_tied_weights_and_grad_reduce(schedule):
    run_ranks(_pp_dp, 4, schedule, timeout_s=240)


def test_pp2_dp2_grad_reduce_then_scale():
    run_ranks(_pp_dp, 4, "1f1b", True, timeout_s=240)


# ---------------------------------------------------------------------------------------------------------------
# Stage modules wrapped by PyTorch's own data-parallel containers (reference test/test_composability.py:203-368:
# DDP | FSDP x gpipe | 1f1b | looped_bfs | interleaved_1f1b on a 2 x 2 mesh; gradients equal the single-process
# gradients averaged over the replicas).  The runtime must keep them from reducing on every microbatch.
D_HID = 16


def _wrapped(rank, world, wrapper, schedule_name):
    import copy

    import torch.distributed as dist
    import torch.nn as nn
    from torch.distributed.device_mesh import DeviceMesh

    import pippy_b200 as pp
    from pippy_b200.parallel.mesh import init_mesh

    mesh = init_mesh(pp_size=2, dp_size=2)
    torch.manual_seed(0)
    n_local = 1 if schedule_name in ("ScheduleGPipe", "Schedule1F1B") else 2
    n_stages = 2 * n_local
    blocks = [nn.Sequential(nn.Linear(D_HID, D_HID), nn.Tanh(), nn.Linear(D_HID, D_HID)) for _ in range(n_stages)]
    reference = copy.deepcopy(nn.Sequential(*blocks))
    n_mb, batch = 4, 8
    gen = torch.Generator().manual_seed(7)
    xs = [torch.randn(batch, D_HID, generator=gen) for _ in range(2)]
    ys = [torch.randn(batch, D_HID, generator=gen) for _ in range(2)]
    x, y = xs[mesh.dp_rank], ys[mesh.dp_rank]

    dp_ranks = dist.get_process_group_ranks(mesh.dp_group)
    stages = []
    for k in range(n_local):
        idx = mesh.pp_rank + 2 * k
        mod = blocks[idx]
        if wrapper == "ddp":
            mod = nn.parallel.DistributedDataParallel(mod, process_group=mesh.dp_group)
        else:
            from torch.distributed.fsdp import fully_shard

            fully_shard(mod, mesh=DeviceMesh.from_group(mesh.dp_group, "cpu", mesh=dp_ranks, mesh_dim_names=("dp",)))
        stages.append(pp.ManualPipelineStage(mod, idx, n_stages, torch.device("cpu"), n_mb,
                                             input_args=torch.empty(batch // n_mb, D_HID), group=mesh.pp_group))
    loss_fn = nn.MSELoss(reduction="sum")
    cls = getattr(pp, schedule_name)
    schedule = cls(stages[0] if n_local == 1 else stages, n_mb, loss_fn=loss_fn)
    first, last = mesh.pp_rank == 0, mesh.pp_rank == 1
    losses = []
    if first and not last:
        schedule.step(x)
    elif last:
        schedule.step(target=y, losses=losses)

    # oracle: the whole model on both replicas' batches; DDP and FSDP average over the replicas
    for d in range(2):
        (loss_fn(reference(xs[d]), ys[d]) / 2).backward()
    for st in stages:
        want = dict(reference[st.stage_index].named_parameters())
        inner = st.submod.module if wrapper == "ddp" else st.submod
        for name, p in inner.named_parameters():
            got = p.grad.full_tensor() if hasattr(p.grad, "full_tensor") else p.grad
            torch.testing.assert_close(got, want[name].grad, rtol=1e-4, atol=1e-5,
                                       msg=f"{wrapper} {schedule_name} stage {st.stage_index} {name}")
    dist.barrier()


@pytest.mark.parametrize("wrapper", ["ddp", "fsdp"])
@pytest.mark.parametrize("schedule_name", ["ScheduleGPipe", "Schedule1F1B", "ScheduleInterleaved1F1B"])
def test_pp2_dp2_with_torch_data_parallel_wrappers(wrapper, schedule_name):
    run_ranks(_wrapped, 4, wrapper, schedule_name, timeout_s=240)


def _llama_v_shape(rank, world):
    """The V-shaped zero-bubble schedule trains the same Llama as the wrap-around one: same loss, same updated
    parameters per stage (stage modules are seeded by stage index, so both placements build identical weights)."""
    import torch.distributed as dist

    from pippy_b200.models.llama import LlamaConfig
    from pippy_b200.train import build_llama_pipeline

    cfg = LlamaConfig(vocab_size=64, dim=32, n_layers=4, n_heads=2, ffn_dim=64)
    B, S, n_mb = 4, 16, 4
    gen = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=gen)
    results = {}
    for schedule in ("zero_bubble", "zbv"):
        pipe = build_llama_pipeline(cfg, B, S, n_mb, torch.device("cpu"), schedule=schedule, virtual_stages=2,
                                    dtype=torch.float32, lr=1e-2, weight_decay=0.0, balance=False)
        assert pipe.holds_first == (rank == 0)
        assert pipe.holds_last == ((rank == 0) if schedule == "zbv" else (rank == world - 1))
        loss = pipe.train_step(inputs=ids if pipe.holds_first else None, target=ids if pipe.holds_last else None)
        state = {st.stage_index: {k: v.detach().clone() for k, v in st.submod.state_dict().items()} for st in pipe.stages}
        results[schedule] = (None if loss is None else float(loss), state)
    # gather every stage's updated parameters and the loss from whichever rank holds them
    gathered = [None] * world
    dist.all_gather_object(gathered, results)
    merged = {sch: {} for sch in ("zero_bubble", "zbv")}
    losses = {}
    for part in gathered:
        for sch, (loss, state) in part.items():
            merged[sch].update(state)
            if loss is not None:
                losses[sch] = loss
    assert sorted(merged["zbv"]) == sorted(merged["zero_bubble"]) == [0, 1, 2, 3]
    assert abs(losses["zbv"] - losses["zero_bubble"]) < 1e-5
    for s in range(4):
        for k, v in merged["zero_bubble"][s].items():
            torch.testing.assert_close(merged["zbv"][s][k], v, rtol=1e-5, atol=1e-6, msg=f"stage {s} {k}")


def test_llama_v_shaped_schedule_matches_wrap_around():
    run_ranks(_llama_v_shape, 2, timeout_s=240)


def _llama_checkpointing(rank, world, schedule):
    """Activation checkpointing changes what is kept, not what is computed: same loss and the same updated
    parameters, also when the weight-gradient passes are deferred (zero-bubble)."""
    import torch.distributed as dist

    from pippy_b200.models.llama import LlamaConfig
    from pippy_b200.train import build_llama_pipeline

    cfg = LlamaConfig(vocab_size=64, dim=32, n_layers=4, n_heads=2, ffn_dim=64)
    B, S, n_mb = 4, 16, 4
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(5))
    out = {}
    for ckpt in (False, True):
        pipe = build_llama_pipeline(cfg, B, S, n_mb, torch.device("cpu"), schedule=schedule, virtual_stages=2,
                                    dtype=torch.float32, lr=1e-2, weight_decay=0.0, activation_checkpointing=ckpt)
        loss = pipe.train_step(inputs=ids if pipe.holds_first else None, target=ids if pipe.holds_last else None)
        out[ckpt] = (None if loss is None else float(loss),
                     [{k: v.detach().clone() for k, v in st.submod.state_dict().items()} for st in pipe.stages])
    if out[False][0] is not None:
        assert abs(out[False][0] - out[True][0]) < 1e-6
    for a, b in zip(out[False][1], out[True][1]):
        for k in a:
            torch.testing.assert_close(b[k], a[k], rtol=1e-5, atol=1e-6, msg=k)
    dist.barrier()


@pytest.mark.parametrize("schedule", ["interleaved_1f1b", "zero_bubble"])
def test_llama_activation_checkpointing_same_result(schedule):
    run_ranks(_llama_checkpointing, 2, schedule, timeout_s=240)


def _gpt2_v_shape(rank, world):
    """GPT-2 with its tied embedding / LM head: on the V shape both ends live on rank 0, so the head simply uses the
    embedding parameter; loss and updated parameters equal the wrap-around schedule's (which syncs the tied pair
    across the first and last rank)."""
    import torch.distributed as dist

    from pippy_b200.models.gpt2 import GPT2Config
    from pippy_b200.train import build_gpt2_pipeline

    cfg = GPT2Config.tiny()
    B, S, n_mb = 4, 16, 4
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(9))
    results = {}
    for schedule in ("zero_bubble", "zbv"):
        pipe = build_gpt2_pipeline(cfg, B, S, n_mb, torch.device("cpu"), schedule=schedule, virtual_stages=2,
                                   dtype=torch.float32, lr=1e-2, weight_decay=0.0)
        if schedule == "zbv":
            assert pipe.holds_first == pipe.holds_last == (rank == 0)
            if rank == 0:
                first = next(s for s in pipe.stages if s.is_first)
                last = next(s for s in pipe.stages if s.is_last)
                assert last.submod.lm_head.weight is first.submod.wte.weight
        loss = pipe.train_step(inputs=ids if pipe.holds_first else None, target=ids if pipe.holds_last else None)
        state = {st.stage_index: {k: v.detach().clone() for k, v in st.submod.state_dict().items()} for st in pipe.stages}
        results[schedule] = (None if loss is None else float(loss), state)
    gathered = [None] * world
    dist.all_gather_object(gathered, results)
    merged, losses = {"zero_bubble": {}, "zbv": {}}, {}
    for part in gathered:
        for sch, (loss, state) in part.items():
            merged[sch].update(state)
            if loss is not None:
                losses[sch] = loss
    assert abs(losses["zbv"] - losses["zero_bubble"]) < 1e-5
    for s in range(4):
        for k, v in merged["zero_bubble"][s].items():
            torch.testing.assert_close(merged["zbv"][s][k], v, rtol=1e-5, atol=1e-6, msg=f"stage {s} {k}")


def test_gpt2_v_shaped_schedule_keeps_tied_weights_on_one_rank():
    run_ranks(_gpt2_v_shape, 2, timeout_s=240)


def _llama_tp_pp(rank, world):
    """Tensor (+ sequence) parallel x pipeline on a 2 x 2 gloo mesh against the same weights gathered into one
    unsharded model: loss, and the gradients of replicated parameters that work on token shards (norm weights,
    embedding: partial sums added over the tensor-parallel group) and of sharded ones (local slices)."""
    import torch.distributed as dist

    from pippy_b200.models.llama import Llama, LlamaConfig, causal_lm_loss
    from pippy_b200.parallel.mesh import init_mesh
    from pippy_b200.train import build_llama_tp_pipeline

    mesh = init_mesh(pp_size=2, tp_size=2)
    cfg = LlamaConfig(vocab_size=96, dim=32, n_layers=2, n_heads=4, ffn_dim=64)
    B, S, n_mb = 4, 8, 2
    pipe = build_llama_tp_pipeline(cfg, B, S, n_mb, torch.device("cpu"), schedule="1f1b", pp_group=mesh.pp_group,
                                   tp_group=mesh.tp_group, dtype=torch.float32, lr=0.0, weight_decay=0.0)
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(21))
    losses = []
    if pipe.holds_first and pipe.holds_last:
        pipe.schedule.step(ids, target=ids, losses=losses)
    elif pipe.holds_first:
        pipe.schedule.step(ids)
    elif pipe.holds_last:
        pipe.schedule.step(target=ids, losses=losses)
    else:
        pipe.schedule.step()
    for hook in pipe.pre_optimizer:
        hook()
    for grp in pipe.optimizer.groups:
        grp.fold_autograd_grads()

    # gather every rank's parameters and gradients and rebuild the unsharded model on every rank
    mine = {f"{mesh.pp_rank}:{mesh.tp_rank}:{n}": (p.detach().clone(), p.main_grad.clone())
            for n, p in pipe.stages[0].submod.named_parameters()}
    everything = [None] * world
    dist.all_gather_object(everything, mine)
    table = {k: v for part in everything for k, v in part.items()}
    hd, H = cfg.head_dim, cfg.n_heads // 2
    full = Llama(cfg, dtype=torch.float32)

    def join(pp, name, which):
        a, b = table[f"{pp}:0:{name}"][which], table[f"{pp}:1:{name}"][which]
        if name.endswith("wqkv.weight"):  # each shard is [q heads | k heads | v heads] of its rank
            qa, ka, va = a.split(H * hd)
            qb, kb, vb = b.split(H * hd)
            return torch.cat([qa, qb, ka, kb, va, vb])
        if name.endswith("w_gate_up.weight"):  # each shard is [gate | up] of its rank
            ga, ua = a.chunk(2)
            gb, ub = b.chunk(2)
            return torch.cat([ga, gb, ua, ub])
        if name.endswith("wo.weight") or name.endswith("w_down.weight"):
            return torch.cat([a, b], dim=1)
        return a  # replicated

    names = {}
    for k in table:
        pp, tpr, name = k.split(":", 2)
        names[name] = int(pp)
    with torch.no_grad():
        for name, p in full.named_parameters():
            key = name.replace("attention.wqkv", "wqkv").replace("attention.wo", "wo") \
                      .replace("feed_forward.w_gate_up", "w_gate_up").replace("feed_forward.w_down", "w_down")
            p.copy_(join(names[key], key, 0))
    total = 0.0
    for mb_ids in ids.chunk(n_mb):
        l = causal_lm_loss(full(mb_ids), mb_ids)
        l.backward()
        total += float(l)
    if losses:
        assert abs(float(torch.stack(losses).sum()) - total) < 1e-4
    for name, p in full.named_parameters():
        key = name.replace("attention.wqkv", "wqkv").replace("attention.wo", "wo") \
                  .replace("feed_forward.w_gate_up", "w_gate_up").replace("feed_forward.w_down", "w_down")
        torch.testing.assert_close(join(names[key], key, 1), p.grad, rtol=1e-4, atol=1e-5, msg=name)
        if not any(key.endswith(t) for t in ("wqkv.weight", "w_gate_up.weight", "wo.weight", "w_down.weight")):
            # replicated parameters carry the same gradient on both tensor-parallel ranks
            torch.testing.assert_close(table[f"{names[key]}:0:{key}"][1], table[f"{names[key]}:1:{key}"][1],
                                       rtol=1e-5, atol=1e-6, msg=name)
    dist.barrier()


def test_llama_tp2_pp2_matches_unsharded_model():
    run_ranks(_llama_tp_pp, 4, timeout_s=240)


def _unit_cut_partitions_match_single_stage(dev):
    """A two-layer Llama cut after EVERY unit of a layer (eight stages on one rank: boundaries after a1 and f1 hand
    over the residual stream together with the attention / SwiGLU output, and the residual stream leaves such a
    stage as the fork of its norm) gives the loss and the gradients of the single-stage model, weight for weight."""
    from pippy_b200.models.llama import LlamaConfig
    from pippy_b200.train import build_llama_pipeline

    cfg = LlamaConfig(vocab_size=1024, dim=512, n_layers=2, n_heads=4, ffn_dim=1024)
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (4, 256), device=dev)
    res, weights = {}, None
    for v, sched in ((1, "1f1b"), (8, "interleaved_1f1b"), (8, "zero_bubble")):
        pipe = build_llama_pipeline(cfg, 4, 256, 2, dev, schedule=sched, virtual_stages=v, seed=11, with_optimizer=True)
        pipe.optimizer = None  # keep the accumulated gradients
        if weights is None:
            weights = {n: p.detach().clone() for st in pipe.stages for n, p in st.submod.named_parameters()}
        else:
            units = [b.units for st in pipe.stages for b in st.submod.layers.values()]
            assert ("a1",) in units and ("f1",) in units, units
            with torch.no_grad():
                for st in pipe.stages:
                    for n, p in st.submod.named_parameters():
                        p.copy_(weights[n])
        loss = float(pipe.train_step(ids, ids))
        grads = {}
        for st in pipe.stages:
            for n, p in st.submod.named_parameters():
                grads[n] = (p.main_grad if p.grad is None else p.grad).float().clone()
        res[(v, sched)] = (loss, grads)
    base_loss, base = res[(1, "1f1b")]
    assert all(g.abs().max().item() > 0 for g in base.values())
    for key in ((8, "interleaved_1f1b"), (8, "zero_bubble")):
        loss, g = res[key]
        assert sorted(g) == sorted(base)
        assert abs(loss - base_loss) < 1e-6, key
        for n in base:
            rel = ((g[n] - base[n]).abs().max() / base[n].abs().max().clamp(min=1e-9)).item()
            assert rel < 1e-3, (key, n, rel)


def test_unit_cut_partitions_match_single_stage():
    _unit_cut_partitions_match_single_stage(torch.device("cpu"))


@pytest.mark.gpu
def test_unit_cut_partitions_match_single_stage_on_the_kernels():
    from pippy_b200.ops import _lib

    _unit_cut_partitions_match_single_stage(torch.device("cuda", 0))
    torch.cuda.synchronize()
    _lib.check_device_errors()
