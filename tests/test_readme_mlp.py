"""README MLP (512->512->1024->256->10) on 2 gloo ranks: loss and gradients equal the unsplit model.
Mirrors the reference's test/test_grad.py and test/test_bwd.py oracle (unsplit model on the last rank)."""
import copy

import pytest
import torch
import torch.nn as nn

from _mp import run_ranks


class MLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.layer0 = nn.Sequential(nn.Linear(512, 512), nn.ReLU())
        self.layer1 = nn.Sequential(nn.Linear(512, 1024), nn.ReLU())
        self.layer2 = nn.Sequential(nn.Linear(1024, 256), nn.ReLU())
        self.layer3 = nn.Linear(256, 10)

    def forward(self, x):
        return self.layer3(self.layer2(self.layer1(self.layer0(x))))


def _stage_modules(model, n):
    layers = [model.layer0, model.layer1, model.layer2, model.layer3]
    per = len(layers) // n
    return [nn.Sequential(*layers[i * per:(i + 1) * per]) for i in range(n)]


def _run(rank, world, schedule_name, v):
    import torch.distributed as dist

    import pippy_b200 as pp

    torch.manual_seed(0)
    model = MLP()
    x = torch.randn(64, 512)
    y = torch.randint(0, 10, (64,))
    loss_fn = nn.CrossEntropyLoss(reduction="sum")
    ref = copy.deepcopy(model)
    ref_loss = loss_fn(ref(x), y)
    ref_loss.backward()

    n_mb = 4
    num_stages = world * v
    mods = _stage_modules(model, num_stages)
    stages = []
    in_dims = {0: 512}
    dims = [512, 512, 1024, 256, 10]
    per = 4 // num_stages
    v_shape = schedule_name == "zbv"  # rank r holds stages r and 2P-1-r
    held = sorted(st for st, r in pp.schedules.v_placement(world).items() if r == rank) if v_shape else \
        [rank + k * world for k in range(v)]
    last_rank = 0 if v_shape else (num_stages - 1) % world
    for s in held:
        inp = torch.empty(64 // n_mb, dims[s * per], device="meta")
        stages.append(pp.ManualPipelineStage(mods[s].to("cpu"), s, num_stages, torch.device("cpu"), n_mb,
                                             input_args=inp.to("cpu") if False else torch.empty(64 // n_mb, dims[s * per])))
    cls = {
        "gpipe": pp.ScheduleGPipe, "1f1b": pp.Schedule1F1B, "bfs": pp.ScheduleLoopedBFS,
        "interleaved": pp.ScheduleInterleaved1F1B, "zb": pp.ScheduleInterleavedZeroBubble,
        "zbv": pp.ScheduleZBVZeroBubble,
    }[schedule_name]
    sched = cls(stages[0] if v == 1 and schedule_name in ("gpipe", "1f1b") else stages, n_mb, loss_fn=loss_fn)
    losses = []
    for it in range(2):  # second iteration checks state is reset between steps
        for st in stages:
            st.submod.zero_grad()
        if rank == 0 and rank == last_rank:
            out = sched.step(x, target=y, losses=losses)
        elif rank == 0:
            out = sched.step(x)
        elif rank == last_rank:
            out = sched.step(target=y, losses=losses)
        else:
            out = sched.step()
    if rank == last_rank:
        torch.testing.assert_close(out, ref(x))
        torch.testing.assert_close(torch.stack(losses).sum(), ref_loss)
    ref_params = dict(ref.named_parameters())
    names = ["layer0.0", "layer1.0", "layer2.0", "layer3"]
    for st in stages:
        s = st.stage_index
        for li, sub in enumerate(st.submod):
            lin = sub[0] if isinstance(sub, nn.Sequential) else sub
            name = names[s * per + li]
            torch.testing.assert_close(lin.weight.grad, ref_params[name + ".weight"].grad)
            torch.testing.assert_close(lin.bias.grad, ref_params[name + ".bias"].grad)
    dist.barrier()


@pytest.mark.parametrize("schedule_name,v", [("gpipe", 1), ("1f1b", 1), ("zb", 1), ("bfs", 2), ("interleaved", 2), ("zb", 2),
                                             ("zbv", 2)])
def test_readme_mlp_two_ranks(schedule_name, v):
    run_ranks(_run, 2, schedule_name, v)
