"""Training step with a loss function and per-microbatch losses (reference examples/basic/example_train.py).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 3 examples/basic/example_train.py [--schedule 1f1b]
"""
import argparse
import os

import torch
import torch.distributed as dist

import pippy_b200 as pp
from pippy_b200.models.mlp import ReadmeMLP

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--schedule", default="gpipe", choices=["gpipe", "1f1b", "zero_bubble"])
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    dist.init_process_group("nccl" if use_cuda else "gloo")
    torch.manual_seed(0)
    model = ReadmeMLP()
    x, target = torch.randn(32, 512), torch.randn(32, 10)
    chunks = 4
    pipe = pp.pipeline(model, chunks, (x,), split_spec={f"layer{i}": pp.SplitPoint.END for i in range(world - 1)})
    stage = pp.PipelineStage(pipe, rank, device)
    cls = {"gpipe": pp.ScheduleGPipe, "1f1b": pp.Schedule1F1B, "zero_bubble": pp.ScheduleZeroBubble}[args.schedule]
    schedule = cls(stage, chunks, loss_fn=torch.nn.MSELoss(reduction="sum"))
    optimizer = torch.optim.SGD(stage.submod.parameters(), lr=0.01)
    for step in range(3):
        optimizer.zero_grad()
        losses = []
        if rank == 0:
            schedule.step(x.to(device))
        elif rank == world - 1:
            schedule.step(target=target.to(device), losses=losses)
            print(f"step {step}: loss {torch.stack(losses).sum().item():.4f}")
        else:
            schedule.step()
        optimizer.step()
    dist.barrier()
    dist.destroy_process_group()
