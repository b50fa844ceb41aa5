"""Hand-written stages: metadata encoding, constructor and input checks, stages with several inputs and outputs,
and two optimizer steps against the unsplit model (reference test/test_pipeline_schedule.py:191-239, 477-541 and
test/test_optim.py:58-99, test/test_grad.py:64-137)."""
import copy

import pytest
import torch
import torch.nn as nn

import pippy_b200 as pp
from pippy_b200.manual_stage import create_metadata_tensor, extract_metadata_from_tensor

from _mp import run_ranks

D = 16


def test_metadata_tensor_roundtrip_and_overflow():
    tensors = [torch.empty(4, 3), torch.empty(()), torch.empty(2, 5, 7), torch.empty(0)]
    md = create_metadata_tensor(tensors)
    assert md.dtype == torch.int32 and md.numel() == 100
    assert extract_metadata_from_tensor(md) == [t.shape for t in tensors]
    assert extract_metadata_from_tensor(create_metadata_tensor([])) == []
    with pytest.raises(ValueError):
        create_metadata_tensor([torch.empty(*([1] * 8)) for _ in range(12)])  # 12 * 9 entries > 100


def test_constructor_rejects_non_tensor_examples():
    with pytest.raises(TypeError):
        pp.ManualPipelineStage(nn.Linear(D, D), 0, 1, torch.device("cpu"), 2, input_args={"x": torch.empty(2, D)})
    with pytest.raises(TypeError):
        pp.ManualPipelineStage(nn.Linear(D, D), 0, 1, torch.device("cpu"), 2, input_args=[torch.empty(2, D), 3])
    with pytest.raises(TypeError):
        pp.ManualPipelineStage(nn.Linear(D, D), 0, 1, torch.device("cpu"), 2, input_args=torch.empty(2, D),
                               output_args="not a tensor")


def test_microbatch_list_checks():
    stage = pp.ManualPipelineStage(nn.Linear(D, D), 0, 1, torch.device("cpu"), 2, input_args=torch.empty(2, D))
    sched = pp.ScheduleGPipe(stage, 2)
    with pytest.raises(TypeError):
        sched._step_microbatches(arg_mbs=(torch.empty(2, D), torch.empty(2, D)))
    with pytest.raises(ValueError):
        sched._step_microbatches(arg_mbs=[(torch.empty(2, D),)])
    with pytest.raises(TypeError):
        sched._step_microbatches(arg_mbs=[(torch.empty(2, D),)] * 2, losses=())


class TwoOut(nn.Module):
    """First stage: one input, two outputs."""

    def __init__(self):
        super().__init__()
        self.a, self.b = nn.Linear(D, D), nn.Linear(D, 2 * D)

    def forward(self, x):
        return torch.relu(self.a(x)), self.b(x)


class TwoIn(nn.Module):
    """Second stage: two inputs, one output."""

    def __init__(self):
        super().__init__()
        self.c, self.d = nn.Linear(D, D), nn.Linear(2 * D, D)

    def forward(self, u, v):
        return self.c(u) + torch.tanh(self.d(v))


class Whole(nn.Module):
    def __init__(self):
        super().__init__()
        self.first, self.second = TwoOut(), TwoIn()

    def forward(self, x):
        return self.second(*self.first(x))


def _two_steps(rank, world, schedule_name):
    torch.manual_seed(0)
    whole = Whole()
    ref = copy.deepcopy(whole)
    n_mb, batch = 4, 8
    part = whole.first if rank == 0 else whole.second
    example = torch.empty(batch // n_mb, D) if rank == 0 else (torch.empty(batch // n_mb, D),
                                                               torch.empty(batch // n_mb, 2 * D))
    stage = pp.ManualPipelineStage(part, rank, world, torch.device("cpu"), n_mb, input_args=example)
    assert stage.init_p2p_neighbors()
    loss_fn = nn.MSELoss(reduction="sum")
    schedule = getattr(pp, schedule_name)(stage, n_mb, loss_fn=loss_fn)
    opt = torch.optim.SGD(part.parameters(), lr=0.05, momentum=0.9)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    for step in range(2):
        g = torch.Generator().manual_seed(100 + step)
        x, y = torch.randn(batch, D, generator=g), torch.randn(batch, D, generator=g)
        opt.zero_grad()
        ref_opt.zero_grad()
        ref_loss = loss_fn(ref(x), y)
        ref_loss.backward()
        losses = []
        if rank == 0:
            schedule.step(x)
        else:
            out = schedule.step(target=y, losses=losses)
            torch.testing.assert_close(out, ref(x), rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(torch.stack(losses).sum(), ref_loss, rtol=1e-4, atol=1e-5)
        ref_part = ref.first if rank == 0 else ref.second
        for (name, p), (_, q) in zip(part.named_parameters(), ref_part.named_parameters()):
            torch.testing.assert_close(p.grad, q.grad, rtol=1e-4, atol=1e-5, msg=f"step {step} grad {name}")
        opt.step()
        ref_opt.step()
    for (name, p), (_, q) in zip(part.named_parameters(), (ref.first if rank == 0 else ref.second).named_parameters()):
        torch.testing.assert_close(p, q, rtol=1e-4, atol=1e-5, msg=f"parameter {name} after two steps")


@pytest.mark.parametrize("schedule_name", ["ScheduleGPipe", "Schedule1F1B"])
def test_multi_input_output_stages_two_sgd_steps(schedule_name):
    run_ranks(_two_steps, 2, schedule_name)
