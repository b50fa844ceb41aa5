"""Forward-only pipeline of the README MLP with tracer-made stages (reference examples/basic/example.py).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 3 examples/basic/example.py
"""
import os

import torch
import torch.distributed as dist

import pippy_b200 as pp
from pippy_b200.models.mlp import ReadmeMLP

if __name__ == "__main__":
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    dist.init_process_group("nccl" if use_cuda else "gloo")
    torch.manual_seed(0)
    model = ReadmeMLP()
    x = torch.randn(32, 512)
    chunks = 4
    split = {f"layer{i}": pp.SplitPoint.END for i in range(world - 1)}
    pipe = pp.pipeline(model, chunks, example_args=(x,), split_spec=split)
    assert pipe.num_stages == world, (pipe.num_stages, world)
    stage = pp.PipelineStage(pipe, rank, device)
    schedule = pp.ScheduleGPipe(stage, chunks)
    out = schedule.step(x.to(device)) if rank == 0 else schedule.step()
    if rank == world - 1:
        torch.testing.assert_close(out.cpu(), model(x), rtol=1e-4, atol=1e-4)
        print("pipeline output equals the unsplit model")
    dist.barrier()
    dist.destroy_process_group()
