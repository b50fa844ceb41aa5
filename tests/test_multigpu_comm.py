"""Fused communication kernels on 2 and 4 GPUs (peer memory over NVLink), each against a plain fp32 reference."""
import pytest
import torch

from _mp import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _need(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")


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
        # the wire format is bf16: peers' contributions and the published sum are each rounded once
        torch.testing.assert_close(flat.grad.cpu(), want, rtol=2e-2, atol=2e-2)
        gathered = [torch.empty_like(flat.grad) for _ in range(world)]
        dist.all_gather(gathered, flat.grad)
        for other in gathered[1:]:
            assert torch.equal(gathered[0], other)  # every replica holds the same bits
    dist.barrier()


@pytest.mark.parametrize("world", [2, 4])
def test_fused_dp_allreduce(world):
    _need(world)
    run_ranks(_dp_allreduce, world, backend="nccl", timeout_s=180)


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


@pytest.mark.parametrize("world", [2, 4])
def test_fused_tp_linears(world):
    _need(world)
    run_ranks(_tp_fused, world, backend="nccl", timeout_s=240)


def _moe_ep(rank, world):
    import torch.distributed as dist

    from pippy_b200.ops import _lib
    from pippy_b200.parallel.ep import EPContext, MoEFeedForward

    dev = torch.device("cuda", rank)
    T, H, Fd, E = 384, 256, 512, 4
    ep = EPContext(None, max_tokens=T, hidden=H, top_k=2, n_experts=E, device=dev)
    torch.manual_seed(5)
    dense = MoEFeedForward(H, Fd, E, 2, None, 1, 0, aux_coef=0.01, device=dev, dtype=torch.bfloat16)  # all experts
    sharded = MoEFeedForward(H, Fd, E, 2, ep, world, rank, aux_coef=0.01, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        sharded.router.copy_(dense.router)
        for i, e in enumerate(sharded.local_experts):
            sharded.w_gate_up[i].copy_(dense.w_gate_up[e])
            sharded.w_down[i].copy_(dense.w_down[e])
    for it in range(2):
        g = torch.Generator(device="cpu").manual_seed(50 + it)
        xs = [torch.randn(T, H, generator=g).bfloat16() for _ in range(world)]   # every rank's tokens
        dys = [torch.randn(T, H, generator=g).bfloat16() for _ in range(world)]
        x = xs[rank].to(dev).requires_grad_()
        for p in sharded.parameters():
            p.grad = None
        out = sharded(x)
        out.backward(dys[rank].to(dev))
        torch.cuda.synchronize()
        _lib.check_device_errors()
        # oracle: the dense layer on this rank's tokens (outputs, input grads) and on all tokens (expert grads)
        for p in dense.parameters():
            p.grad = None
        xr = xs[rank].to(dev).requires_grad_()
        ref = dense(xr)
        ref.backward(dys[rank].to(dev))
        rel = lambda a, b: ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6)).item()
        assert rel(out, ref) < 2e-2, ("out", rel(out, ref))
        assert rel(x.grad, xr.grad) < 2e-2, ("dx", rel(x.grad, xr.grad))
        assert rel(sharded.router.grad[:E], dense.router.grad[:E]) < 3e-2, ("drouter", rel(sharded.router.grad, dense.router.grad))
        for other in range(world):
            if other != rank:
                xo = xs[other].to(dev)
                dense(xo).backward(dys[other].to(dev))
        for i, e in enumerate(sharded.local_experts):
            assert rel(sharded.w_down.grad[i], dense.w_down.grad[e]) < 2e-2, ("dWdown", e)
            assert rel(sharded.w_gate_up.grad[i], dense.w_gate_up.grad[e]) < 2e-2, ("dWgu", e)
    dist.barrier()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_moe(world):
    _need(world)
    run_ranks(_moe_ep, world, backend="nccl", timeout_s=240)
