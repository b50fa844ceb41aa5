"""Experts placed on pipeline stages: a pre-processing stage fans out to one stage per expert, the last stage
concatenates (reference examples/mixture_of_experts/dist_moe.py).  The fan-out makes every expert stage read the
same activation, i.e. forward skip connections; this runtime also sends the gradients back along them, so the
example trains, which the reference's does not.  For real expert parallelism (router, top-2, all-to-all) see
examples/mixtral/train_mixtral_pp_ep.py.

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 5 examples/mixture_of_experts/experts_as_stages.py
"""
import copy
import os

import torch
import torch.distributed as dist
import torch.nn as nn

import pippy_b200 as pp

D_HID, BATCH = 16, 8


class Expert(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.up, self.down = nn.Linear(d, d), nn.Linear(d, d)

    def forward(self, x):
        return self.down(torch.relu(self.up(x)))


class ExpertsSideBySide(nn.Module):
    def __init__(self, n_experts):
        super().__init__()
        self.pre_proc = nn.Linear(D_HID, D_HID)
        self.experts = nn.ModuleList(Expert(D_HID) for _ in range(n_experts))

    def forward(self, x):
        x = self.pre_proc(x)
        return torch.cat([e(x) for e in self.experts], dim=1)


if __name__ == "__main__":
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    dist.init_process_group("nccl" if use_cuda else "gloo")
    torch.manual_seed(0)
    n_experts = world - 2                      # pre-processing stage + experts + concatenation stage
    model = ExpertsSideBySide(n_experts)
    unsplit = copy.deepcopy(model)             # the stages take over `model`'s parameters; compare against a copy
    x, target = torch.randn(BATCH, D_HID), torch.randn(BATCH, D_HID * n_experts)

    split = {"pre_proc": pp.SplitPoint.END}
    split.update({f"experts.{i}": pp.SplitPoint.END for i in range(n_experts)})
    chunks = 2
    pipe = pp.pipeline(model, chunks, example_args=(x,), split_spec=split)
    assert pipe.num_stages == world, (pipe.num_stages, world)
    torch.testing.assert_close(pipe(x)[0], unsplit(x))

    stage = pp.PipelineStage(pipe, rank, device)
    loss_fn = nn.MSELoss(reduction="sum")
    schedule = pp.ScheduleGPipe(stage, chunks, loss_fn=loss_fn)
    losses = []
    if rank == 0:
        schedule.step(x.to(device))
    elif rank == world - 1:
        out = schedule.step(target=target.to(device), losses=losses)
        torch.testing.assert_close(out.cpu(), unsplit(x), rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(torch.stack(losses).sum().cpu(), loss_fn(unsplit(x), target), rtol=1e-4, atol=1e-4)
        print("experts-as-stages: output and loss equal the unsplit model")
    else:
        schedule.step()

    # Gradients flowed back through the fan-out: compare this stage's parameters with the unsplit model's.
    loss_fn(unsplit(x), target).backward()
    want = dict(unsplit.named_parameters())
    for name, p in stage.submod.named_parameters():
        torch.testing.assert_close(p.grad.cpu(), want[name].grad, rtol=1e-3, atol=1e-4)
    print(f"rank {rank}: parameter gradients equal the unsplit model's")
    dist.barrier()
    dist.destroy_process_group()
