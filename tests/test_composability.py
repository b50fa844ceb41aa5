"""Pipeline x data parallel composition on a 2 x 2 gloo mesh: GPT-2 stages with a tied embedding / LM head, stage
gradients reduced at the schedule's REDUCE_GRAD action (reference test/test_composability.py: grads equal the
single-process grads averaged over the replicas)."""
import pytest
import torch

from _mp import run_ranks


def _pp_dp(rank, world, schedule):
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
            torch.testing.assert_close(p.main_grad, want, rtol=2e-4, atol=2e-5, msg=f"{schedule} stage {st.stage_index} {k}")
    dist.barrier()


@pytest.mark.parametrize("schedule", ["1f1b", "zero_bubble"])
def test_pp2_dp2_gpt2_tied_weights_and_grad_reduce(schedule):
    run_ranks(_pp_dp, 4, schedule, timeout_s=240)
