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


def _tp_fused(rank, world):
    import torch.distributed as dist

    from pippy_b200.ops import _lib
    from pippy_b200.parallel.tp import ColumnParallelLinear, RowParallelLinear, TPContext

    dev = torch.device("cuda", rank)
    torch.manual_seed(1)  # same values on every rank, then sliced
    rows, d, ffn = 512, 1024, 1536
    T = rows * world
    tp = TPContext(None, max_rows=rows, max_cols=max(d, ffn), device=dev)
    x_full = torch.randn(T, d, device=dev).bfloat16()
    w_col_full = (torch.randn(ffn, d, device=dev) * 0.03).bfloat16()
    w_row_full = (torch.randn(d, ffn, device=dev) * 0.03).bfloat16()
    res_full = torch.randn(T, d, device=dev).bfloat16()
    dout_full = torch.randn(T, d, device=dev).bfloat16()
    sl = slice(rank * rows, (rank + 1) * rows)
    col = ColumnParallelLinear(d, ffn, tp, world, device=dev, dtype=torch.bfloat16)
    row = RowParallelLinear(ffn, d, tp, world, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        col.weight.copy_(w_col_full[rank * (ffn // world):(rank + 1) * (ffn // world)])
        row.weight.copy_(w_row_full[:, rank * (ffn // world):(rank + 1) * (ffn // world)])
    for it in range(2):  # the second pass exercises workspace and flag reuse
        col.weight.grad = row.weight.grad = None
        x_shard = x_full[sl].clone().requires_grad_()
        res = res_full[sl].clone().requires_grad_()
        h = col(x_shard)                       # [T, ffn/world]
        out = row(torch.relu(h), res)          # [T/world, d]
        out.backward(dout_full[sl])
        torch.cuda.synchronize()
        _lib.check_device_errors()
        # oracle: the unsharded computation in fp32
        xf = x_full.float().requires_grad_()
        wc, wr = w_col_full.float().requires_grad_(), w_row_full.float().requires_grad_()
        ref = torch.relu(xf @ wc.t()).bfloat16().float() @ wr.t() + res_full.float()
        ref.backward(dout_full.float())
        rel = lambda a, b: ((a.float() - b).abs().max() / b.abs().max()).item()
        assert rel(out, ref[sl].detach()) < 2e-2, ("out", it, rel(out, ref[sl].detach()))
        assert rel(x_shard.grad, xf.grad[sl]) < 3e-2, ("dx", it, rel(x_shard.grad, xf.grad[sl]))
        assert rel(res.grad, dout_full[sl].float()) < 1e-3
        cs = slice(rank * (ffn // world), (rank + 1) * (ffn // world))
        assert rel(col.weight.grad, wc.grad[cs]) < 3e-2, ("dWcol", it, rel(col.weight.grad, wc.grad[cs]))
        assert rel(row.weight.grad, wr.grad[:, cs]) < 3e-2, ("dWrow", it, rel(row.weight.grad, wr.grad[:, cs]))
    dist.barrier()


def test_fused_tp_linears_two_gpus():
    run_ranks(_tp_fused, 2, backend="nccl", timeout_s=240)
