"""Pipeline over NCCL on 2 GPUs: same losses as the same stages run on one GPU (needs >= 2 B200s)."""
import pytest
import torch

from _mp import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _losses(device, schedule, virtual, steps=3):
    from pippy_b200.models.llama import LlamaConfig
    from pippy_b200.ops import _lib
    from pippy_b200.train import build_llama_pipeline

    cfg = LlamaConfig(vocab_size=1024, dim=512, n_layers=4, n_heads=4, ffn_dim=1024)
    pipe = build_llama_pipeline(cfg, global_batch=8, seq_len=256, n_microbatches=4, device=device, schedule=schedule,
                                virtual_stages=virtual, lr=1e-3, seed=7)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (8, 256), generator=g).to(device)
    out = []
    for _ in range(steps):
        loss = pipe.train_step(ids if pipe.holds_first else None, ids if pipe.holds_last else None)
        out.append(None if loss is None else float(loss.item()))
    torch.cuda.synchronize()
    _lib.check_device_errors()
    return out, pipe


def _two_ranks(rank, world, expected):
    device = torch.device("cuda", rank)
    for schedule in ("interleaved_1f1b", "zero_bubble"):
        got, pipe = _losses(device, schedule, 2)
        if pipe.holds_last:
            for a, b in zip(got, expected):
                assert abs(a - b) < 2e-2 * abs(b), (schedule, got, expected)
            assert got[-1] < got[0]


def test_two_gpu_pipeline_matches_single_gpu():
    torch.cuda.set_device(0)
    expected, _ = _losses(torch.device("cuda", 0), "interleaved_1f1b", 4)
    run_ranks(_two_ranks, 2, expected, backend="nccl", timeout_s=240)


def _gpt2_losses_single(device, steps):
    """GPT-2 on one GPU over the whole batch: what PP2 x DP2 must reproduce."""
    from pippy_b200.models.gpt2 import GPT2Config
    from pippy_b200.train import build_gpt2_pipeline

    cfg = GPT2Config(vocab_size=1000, n_positions=128, dim=256, n_layers=4, n_heads=4)
    pipe = build_gpt2_pipeline(cfg, 8, 128, 4, device, schedule="interleaved_1f1b", virtual_stages=2, lr=1e-3, seed=3)
    g = torch.Generator().manual_seed(17)
    ids = torch.randint(0, cfg.vocab_size, (8, 128), generator=g).to(device)
    return [float(pipe.train_step(ids, ids)) for _ in range(steps)]


def _gpt2_pp2_dp2(rank, world, expected):
    """Two pipeline ranks x two replicas with the FUSED gradient all-reduce under 1F1B: the mean of the replicas'
    losses follows the single-GPU run on the whole batch step by step (same updates), and the tied embedding /
    LM head stays identical on the first and last pipeline rank."""
    import torch.distributed as dist

    from pippy_b200.models.gpt2 import GPT2Config
    from pippy_b200.ops import _lib
    from pippy_b200.parallel.mesh import init_mesh
    from pippy_b200.train import build_gpt2_pipeline

    device = torch.device("cuda", rank)
    mesh = init_mesh(pp_size=2, dp_size=2)
    cfg = GPT2Config(vocab_size=1000, n_positions=128, dim=256, n_layers=4, n_heads=4)
    pipe = build_gpt2_pipeline(cfg, 4, 128, 2, device, schedule="1f1b", group=mesh.pp_group, dp_group=mesh.dp_group,
                               lr=1e-3, seed=3)
    assert pipe.schedule.grad_reducer is not None and pipe.schedule.grad_reducer.fused
    g = torch.Generator().manual_seed(17)
    ids = torch.randint(0, cfg.vocab_size, (8, 128), generator=g)[mesh.dp_rank * 4:(mesh.dp_rank + 1) * 4].to(device)
    for step in range(len(expected)):
        loss = pipe.train_step(ids if pipe.holds_first else None, ids if pipe.holds_last else None)
        t = torch.tensor([float(loss) if loss is not None else 0.0], device=device)
        dist.all_reduce(t)  # the two last-stage ranks hold one replica's loss each
        got = float(t) / 2
        assert abs(got - expected[step]) < 2e-2 * abs(expected[step]), (step, got, expected)
    torch.cuda.synchronize()
    _lib.check_device_errors()
    # replicas hold the same parameters bit for bit (identical reduced gradients, identical updates)
    flat = pipe.flat.data
    peers = [torch.empty_like(flat) for _ in range(2)]
    dist.all_gather(peers, flat, group=mesh.dp_group)
    assert torch.equal(peers[0], peers[1])


def test_four_gpu_gpt2_pp2_dp2_fused_reducer():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 CUDA devices")
    torch.cuda.set_device(0)
    expected = _gpt2_losses_single(torch.device("cuda", 0), 3)
    run_ranks(_gpt2_pp2_dp2, 4, expected, backend="nccl", timeout_s=300)
