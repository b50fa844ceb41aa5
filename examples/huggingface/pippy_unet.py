"""A small 2-D UNet cut in the middle: skip connections across the cut and a non-tensor argument (reference
examples/huggingface/pippy_unet.py pipelines diffusers' UNet2DModel, split at `mid_block` END, called with
`timestep=1`).  The model here is written out in plain PyTorch so that the example needs no extra package: two
down blocks, a middle block and two up blocks that take the matching down block's output, so the first stage sends
three tensors to the second, and the integer timestep is burnt into the traced program like any non-tensor input.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/huggingface/pippy_unet.py
"""
import copy
import math
import os

import torch
import torch.distributed as dist
import torch.nn as nn

import pippy_b200 as pp


class Block(nn.Module):
    def __init__(self, c_in, c_out, t_dim):
        super().__init__()
        self.conv1 = nn.Conv2d(c_in, c_out, 3, padding=1)
        self.conv2 = nn.Conv2d(c_out, c_out, 3, padding=1)
        self.t_proj = nn.Linear(t_dim, c_out)
        self.norm = nn.GroupNorm(4, c_out)

    def forward(self, x, t_emb):
        h = torch.nn.functional.silu(self.conv1(x)) + self.t_proj(t_emb)[:, :, None, None]
        return torch.nn.functional.silu(self.norm(self.conv2(h)))


class TinyUNet(nn.Module):
    def __init__(self, channels=3, width=16, t_dim=32):
        super().__init__()
        self.t_dim = t_dim
        self.t_mlp = nn.Sequential(nn.Linear(t_dim, t_dim), nn.SiLU(), nn.Linear(t_dim, t_dim))
        self.down1 = Block(channels, width, t_dim)
        self.down2 = Block(width, 2 * width, t_dim)
        self.pool = nn.AvgPool2d(2)
        self.mid_block = Block(2 * width, 2 * width, t_dim)
        self.up2 = Block(4 * width, width, t_dim)
        self.up1 = Block(2 * width, width, t_dim)
        self.out = nn.Conv2d(width, channels, 1)

    def time_embedding(self, timestep: int, batch: int, device):
        half = self.t_dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=device) / half)
        ang = float(timestep) * freqs
        return torch.cat([ang.sin(), ang.cos()]).expand(batch, -1)

    def forward(self, sample, timestep: int = 0):
        t_emb = self.t_mlp(self.time_embedding(timestep, sample.shape[0], sample.device))
        d1 = self.down1(sample, t_emb)
        d2 = self.down2(self.pool(d1), t_emb)
        m = self.mid_block(self.pool(d2), t_emb)
        u2 = self.up2(torch.cat([torch.nn.functional.interpolate(m, scale_factor=2.0), d2], dim=1), t_emb)
        u1 = self.up1(torch.cat([torch.nn.functional.interpolate(u2, scale_factor=2.0), d1], dim=1), t_emb)
        return self.out(u1)


if __name__ == "__main__":
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    assert world == 2, "this example cuts the UNet into two stages"
    use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    dist.init_process_group("nccl" if use_cuda else "gloo")
    torch.manual_seed(0)
    model = TinyUNet().eval()
    unsplit = copy.deepcopy(model)
    chunks, batch = 2, 4
    x = torch.randn(batch, 3, 16, 16)

    pipe = pp.pipeline(model, chunks, example_args=(x,), example_kwargs={"timestep": 1},
                       split_spec={"mid_block": pp.SplitPoint.END})
    assert pipe.num_stages == world
    stage = pp.PipelineStage(pipe, rank, device)
    schedule = pp.ScheduleGPipe(stage, chunks)
    if rank == 0:
        schedule.step(x.to(device), timestep=1)
    else:
        out = schedule.step()
        with torch.no_grad():
            ref = torch.cat([unsplit(x[i * 2:(i + 1) * 2], timestep=1) for i in range(chunks)])
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4)
        n_inputs = sum(1 for s in stage.input_specs if s.source == 0)
        print(f"unet: second stage receives {n_inputs} tensors from the first (skip connections); output equals "
              "the unsplit model")
    dist.barrier()
    dist.destroy_process_group()
