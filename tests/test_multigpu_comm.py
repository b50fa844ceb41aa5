"""Fused communication kernels on 2 GPUs (peer memory over NVLink), each against a plain fp32 reference."""
import pytest
import torch

from _mp import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _dp_allreduce(rank, world):
    import torch.distributed as dist
    import torch.nn as nn

    from pippy_b200.ops import _lib
    from pippy_b200.optim import FlatParams
    from pippy_b200.parallel.dp import GradReducer

    dev = torch.device("cuda", rank)
    torch.manual_seed(0)
    params = [nn.Parameter(torch.zeros(1000, 333, device=dev, dtype=torch.bfloat16)),
              nn.Parameter(torch.zeros(77, device=dev, dtype=torch.bfloat16))]
    flat = FlatParams(params)
    red = GradReducer(flat, None)
    assert red.fused
    for it in range(3):
        g = torch.Generator(device="cpu").manual_seed(100 + it)
        per_rank = [torch.randn(flat.numel, generator=g) for _ in range(world)]
        flat.grad.copy_(per_rank[rank])
        red.reduce_all()
        red.finish()
        torch.cuda.synchronize()
        _lib.check_device_errors()
        want = sum(per_rank) / world
        # owned slice is an exact fp32 sum of bf16-rounded peers + own fp32; others come back through bf16
        torch.testing.assert_close(flat.grad.cpu(), want, rtol=2e-2, atol=2e-2)
        mine = flat.grad.cpu()
        gathered = [torch.empty_like(flat.grad) for _ in range(world)]
        dist.all_gather(gathered, flat.grad)
        torch.testing.assert_close(gathered[0], gathered[1], rtol=1e-2, atol=1e-2)
    dist.barrier()


def test_fused_dp_allreduce_two_gpus():
    run_ranks(_dp_allreduce, 2, backend="nccl", timeout_s=180)
