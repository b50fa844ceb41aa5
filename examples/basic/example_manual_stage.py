"""Hand-written stage modules, no tracing (reference examples/basic/example_manual_stage.py).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 3 examples/basic/example_manual_stage.py
"""
import os

import torch
import torch.distributed as dist
import torch.nn as nn

import pippy_b200 as pp

if __name__ == "__main__":
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    assert world == 3, "this example has three hand-written stages"
    use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    dist.init_process_group("nccl" if use_cuda else "gloo")
    torch.manual_seed(rank)
    chunks, batch = 4, 32
    dims = [512, 512, 1024, 10]
    module = nn.Sequential(nn.Linear(dims[rank], dims[rank + 1]), nn.ReLU() if rank < 2 else nn.Identity()).to(device)
    example_in = torch.empty(batch // chunks, dims[rank], device=device)
    stage = pp.ManualPipelineStage(module, rank, world, device, chunks, input_args=example_in)
    pp.validate_stage_shapes([stage])
    schedule = pp.ScheduleGPipe(stage, chunks)
    out = schedule.step(torch.randn(batch, 512, device=device)) if rank == 0 else schedule.step()
    if rank == world - 1:
        print("output", tuple(out.shape))
    dist.barrier()
    dist.destroy_process_group()
