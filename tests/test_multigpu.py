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
