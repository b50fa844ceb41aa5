"""Trace on CPU, run the stages on GPUs: factory ops traced with ``device=cpu`` are rewritten to the stage's device
(reference examples/cpu_init/gpt2_cpu_init.py).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/cpu_init/cpu_init.py
"""
import os

import torch
import torch.distributed as dist
import torch.nn as nn

import pippy_b200 as pp


class WithFactoryOps(nn.Module):
    def __init__(self):
        super().__init__()
        self.a, self.b = nn.Linear(64, 64), nn.Linear(64, 64)

    def forward(self, x):
        x = self.a(x) + torch.ones(64, device=x.device)
        pp.pipe_split()
        return self.b(x) + torch.arange(64, device=x.device, dtype=x.dtype)


if __name__ == "__main__":
    rank = int(os.environ["RANK"])
    cuda = torch.cuda.is_available() and torch.cuda.device_count() >= 2
    dist.init_process_group("nccl" if cuda else "gloo")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if cuda else torch.device("cpu")
    torch.manual_seed(0)
    model = WithFactoryOps()  # lives on the CPU while it is traced
    x = torch.randn(8, 64)
    pipe = pp.pipeline(model, 2, (x,))
    stage = pp.PipelineStage(pipe, rank, device)  # moves parameters and rewrites the traced devices
    schedule = pp.ScheduleGPipe(stage, 2)
    out = schedule.step(x.to(device)) if rank == 0 else schedule.step()
    if rank == 1:
        torch.testing.assert_close(out.cpu(), model(x), rtol=1e-4, atol=1e-4)
        print("CPU-traced pipeline ran on", device)
    dist.barrier()
    dist.destroy_process_group()
