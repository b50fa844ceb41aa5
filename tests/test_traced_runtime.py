"""Tracer-backed stages driven by every schedule on gloo ranks; oracle = the unsplit model
(reference test/test_fwd.py, test_bwd.py, test_grad.py, test_skip_conn.py, test_interleave.py,
test_pipeline_schedule.py's timing-perturbation and validation cases)."""
import copy
import random
import time

import pytest
import torch
import torch.nn as nn

from _mp import run_ranks

D = 64


class ExampleCode(nn.Module):
    def __init__(self):
        super().__init__()
        self.mm_param = nn.Parameter(torch.randn(D, D) * 0.1)
        self.mm_param2 = nn.Parameter(torch.randn(D, D) * 0.1)
        self.lin = nn.Linear(D, D)
        self.lin2 = nn.Linear(D, D)
        self.register_buffer("buffer", torch.randn(D) * 0.1)

    def forward(self, x, y=torch.zeros(32, D)):
        from pippy_b200 import ir

        x = torch.mm(x, self.mm_param)
        skip = x
        x = torch.relu(x + y)
        ir.pipe_split()
        x = torch.mm(x, self.mm_param) + self.buffer  # mm_param is used by two stages (a tied weight)
        x = self.lin(x)
        ir.pipe_split()
        x = torch.relu(x)
        x = torch.mm(x, self.mm_param2)
        ir.pipe_split()
        x = self.lin2(x) + skip  # skip connection from stage 0 to stage 3
        return torch.relu(x)


def _grads_by_fqn(mod):
    return {k: p.grad for k, p in mod.named_parameters() if p.grad is not None}


def _world4(rank, world):
    import torch.distributed as dist

    import pippy_b200 as pp
    from pippy_b200.ir import pipeline
    from pippy_b200.parallel.tied import TiedParamSync
    from pippy_b200.pipeline_stage import PipelineStage

    torch.manual_seed(0)
    mod = ExampleCode()
    ref = copy.deepcopy(mod)
    x, y, target = torch.randn(32, D), torch.randn(32, D), torch.randn(32, D)
    chunks = 4
    pipe = pipeline(mod, chunks, (x,), {"y": y})
    assert pipe.num_stages == world
    assert pipe.replicated_params == [{"submod_0": "mm_param", "submod_1": "mm_param"}]
    stage = PipelineStage(pipe, rank, torch.device("cpu"))
    assert stage.global_dests[0] == [1, 3], stage.global_dests
    tied = TiedParamSync(pipe, [stage])
    loss_fn = nn.MSELoss(reduction="sum")
    ref_out = ref(x, y)
    ref_loss = loss_fn(ref_out, target)
    ref_loss.backward()
    ref_grads = _grads_by_fqn(ref)

    for name, cls in (("gpipe", pp.ScheduleGPipe), ("1f1b", pp.Schedule1F1B), ("zb", pp.ScheduleZeroBubble)):
        sched = cls(stage, chunks, loss_fn=loss_fn)
        for it in range(2):
            stage.submod.zero_grad()
            losses = []
            if rank == 0:
                out = sched.step(x, y=y)
            elif rank == world - 1:
                out = sched.step(target=target, losses=losses)
            else:
                out = sched.step()
            tied.sync()
        if rank == world - 1:
            torch.testing.assert_close(out, ref_out, msg=name)
            torch.testing.assert_close(torch.stack(losses).sum(), ref_loss, msg=name)
        else:
            assert out is None
        for k, p in stage.submod.named_parameters():
            torch.testing.assert_close(p.grad, ref_grads[k], msg=f"{name}:{k}")

    # forward-only with timing perturbation: random sleeps must not deadlock or change the result
    class Sleepy(nn.Module):
        def __init__(self, inner):
            super().__init__()
            self.inner = inner

        def forward(self, *a, **k):
            time.sleep(random.random() * 0.02 * (1 + rank))
            return self.inner(*a, **k)

    stage.submod = Sleepy(stage.submod)
    sched = pp.Schedule1F1B(stage, chunks, loss_fn=loss_fn)
    if rank == 0:
        sched.step(x, y=y)
    elif rank == world - 1:
        out = sched.step(target=target, losses=[])
        torch.testing.assert_close(out, ref_out)
    else:
        sched.step()
    dist.barrier()


def test_traced_pipeline_four_ranks_skip_tied_all_schedules():
    run_ranks(_world4, 4, timeout_s=240)


class Deep(nn.Module):
    def __init__(self, n=8):
        super().__init__()
        self.layers = nn.ModuleList([nn.Sequential(nn.Linear(D, D), nn.Tanh()) for _ in range(n)])

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x


def _world2(rank, world, tmpdir):
    import os

    import torch.distributed as dist

    import pippy_b200 as pp
    from pippy_b200.checkpoint import CKPT_INDEX_JSON_FILENAME, load_checkpoint, save_checkpoint
    from pippy_b200.ir import SplitPoint, pipeline
    from pippy_b200.manual_stage import ManualPipelineStage, get_stage_shapes, validate_stage_shapes
    from pippy_b200.pipeline_stage import PipelineStage

    torch.manual_seed(0)
    mod = Deep(8)
    ref = copy.deepcopy(mod)
    x, target = torch.randn(16, D), torch.randn(16, D)
    loss_fn = nn.MSELoss(reduction="sum")
    ref_out = ref(x)
    ref_loss = loss_fn(ref_out, target)
    ref_loss.backward()
    ref_grads = _grads_by_fqn(ref)
    n_mb = 4
    pipe = pipeline(mod, n_mb, (x,), split_spec={f"layers.{i}": SplitPoint.BEGINNING for i in (2, 4, 6)})
    assert pipe.num_stages == 4
    stages = [PipelineStage(pipe, rank + k * world, torch.device("cpu")) for k in range(2)]

    for name, cls in (("bfs", pp.ScheduleLoopedBFS), ("interleaved", pp.ScheduleInterleaved1F1B),
                      ("zb", pp.ScheduleInterleavedZeroBubble)):
        sched = cls(stages, n_mb, loss_fn=loss_fn, record_timing=True)
        for st in stages:
            st.submod.zero_grad()
        losses = []
        if rank == 0:
            out = sched.step(x)
        else:
            out = sched.step(target=target, losses=losses)
        if rank == 1:
            torch.testing.assert_close(out, ref_out, rtol=1e-4, atol=1e-5, msg=name)
            torch.testing.assert_close(torch.stack(losses).sum(), ref_loss, rtol=1e-4, atol=1e-4, msg=name)
        for st in stages:
            for k, p in st.submod.named_parameters():
                torch.testing.assert_close(p.grad, ref_grads[k], rtol=1e-4, atol=1e-5, msg=f"{name}:{k}")
        assert 0.0 <= sched.last_step_stats["bubble"] < 1.0 and sched.last_step_stats["per_op_s"]

    # interleaving constraints
    with pytest.raises(ValueError, match="multiple of the"):
        pp.ScheduleInterleaved1F1B(stages, 3, loss_fn=loss_fn)
    with pytest.raises(ValueError):
        pp.ScheduleInterleaved1F1B([stages[0]], n_mb)
    # _check_inputs contract
    sched = pp.ScheduleInterleaved1F1B(stages, n_mb, loss_fn=loss_fn)
    with pytest.raises(TypeError):
        sched._step_microbatches(arg_mbs=(1, 2, 3, 4))
    with pytest.raises(ValueError):
        sched._step_microbatches(arg_mbs=[(), ()])
    with pytest.raises(TypeError):
        sched._step_microbatches(losses=3)

    # ---- checkpoint: every rank saves its two stages, then the files load into the unsplit model and other splits
    ckpt = os.path.join(tmpdir, "ckpt")
    save_checkpoint(stages, ckpt)
    dist.barrier()
    files = sorted(os.listdir(ckpt))
    assert files == sorted([CKPT_INDEX_JSON_FILENAME, "pytorch_model-00001-of-00002.bin", "pytorch_model-00002-of-00002.bin"]), files
    fresh = Deep(8)
    load_checkpoint(fresh, os.path.join(ckpt, CKPT_INDEX_JSON_FILENAME))
    for k, v in fresh.state_dict().items():
        torch.testing.assert_close(v, ref.state_dict()[k])
    other = pipeline(Deep(8), n_mb, (x,), split_spec={"layers.5": SplitPoint.BEGINNING})
    sub = other.get_stage_module(rank)
    load_checkpoint(sub, os.path.join(ckpt, CKPT_INDEX_JSON_FILENAME))
    for k, v in sub.state_dict().items():
        torch.testing.assert_close(v, ref.state_dict()[k])

    # ---- manual stages: shape discovery and validation
    halves = [nn.Sequential(*[copy.deepcopy(ref.layers[i]) for i in range(rank * 4, rank * 4 + 4)])]
    shapes = get_stage_shapes(halves, [rank], 2, rank, world, torch.device("cpu"), microbatch=torch.randn(4, D))
    assert shapes[rank]["inputs"] == [torch.Size([4, D])] and shapes[rank]["outputs"] == [torch.Size([4, D])]
    good = ManualPipelineStage(halves[0], rank, 2, torch.device("cpu"), n_mb, input_args=torch.randn(4, D))
    validate_stage_shapes([good])
    bad_in = torch.randn(4, D) if rank == 0 else torch.randn(4, D + 1)
    bad_mod = halves[0] if rank == 0 else nn.Linear(D + 1, D)
    bad = ManualPipelineStage(bad_mod, rank, 2, torch.device("cpu"), n_mb, input_args=bad_in)
    with pytest.raises(ValueError, match="do not match"):
        validate_stage_shapes([bad])
    with pytest.raises(ValueError):
        validate_stage_shapes([])
    with pytest.raises(TypeError, match="cannot create empty tensors"):
        ManualPipelineStage(halves[0], rank, 2, torch.device("cpu"), n_mb, input_args={"x": 1})
    with pytest.raises(ValueError):
        ManualPipelineStage(halves[0], 2, 2, torch.device("cpu"), n_mb, input_args=torch.randn(4, D))
    good.init_p2p_neighbors()
    dist.barrier()


def test_traced_pipeline_two_ranks_interleaved_checkpoint_validation(tmp_path):
    run_ranks(_world2, 2, str(tmp_path), timeout_s=240)


def _failing(rank, world):
    """A rank that never joins the step: its neighbour's bounded wait must end with ScheduleTimeout."""
    import torch.distributed as dist

    import pippy_b200 as pp
    from pippy_b200.manual_stage import ManualPipelineStage
    from pippy_b200.schedules import ScheduleTimeout

    mod = nn.Linear(D, D)
    stage = ManualPipelineStage(mod, rank, world, torch.device("cpu"), 2, input_args=torch.randn(2, D))
    sched = pp.ScheduleGPipe(stage, 2, p2p_timeout_s=1.5)
    if rank == 0:
        time.sleep(4.0)  # host-side fault: this rank is "stuck" and never sends
    else:
        t0 = time.time()
        with pytest.raises(ScheduleTimeout, match="1RECV_F0|1F0"):
            sched.step()
        assert time.time() - t0 < 3.5


def test_stalled_neighbour_is_detected_by_bounded_wait():
    run_ranks(_failing, 2, timeout_s=60)


def _v_shape_traced(rank, world):
    """Traced stages on the V-shaped placement (rank r holds stages r and 2P-1-r): output, summed loss and every
    parameter gradient equal the unsplit model; the input/weight gradient split runs through the generic
    autograd-graph path because the stages are plain torch modules."""
    import copy

    import torch.nn as nn

    import pippy_b200 as pp

    torch.manual_seed(0)
    model = nn.Sequential(*[nn.Sequential(nn.Linear(16, 16), nn.Tanh()) for _ in range(2 * world)])
    ref = copy.deepcopy(model)
    x, y = torch.randn(8, 16), torch.randn(8, 16)
    pipe = pp.pipeline(model, 4, example_args=(x,), split_spec={str(i): pp.SplitPoint.END for i in range(2 * world - 1)})
    placement = pp.schedules.v_placement(world)
    stages = [pp.PipelineStage(pipe, s, torch.device("cpu")) for s, r in sorted(placement.items()) if r == rank]
    loss_fn = nn.MSELoss(reduction="sum")
    sched = pp.ScheduleZBVZeroBubble(stages, 4, loss_fn=loss_fn)
    losses = []
    if rank == 0:  # first and last stage
        out = sched.step(x, target=y, losses=losses)
        torch.testing.assert_close(out, ref(x), rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(torch.stack(losses).sum(), loss_fn(ref(x), y), rtol=1e-4, atol=1e-5)
    else:
        assert sched.step() is None
    loss_fn(ref(x), y).backward()
    want = dict(ref.named_parameters())
    for st in stages:
        for n, p in st.submod.named_parameters():
            torch.testing.assert_close(p.grad, want[n].grad, rtol=1e-4, atol=1e-5, msg=n)
    with pytest.raises(ValueError):
        stages[0].set_placement({s: 0 for s in range(2 * world)} if rank else {s: 1 for s in range(2 * world)})


def test_traced_stages_on_v_shaped_placement_three_ranks():
    run_ranks(_v_shape_traced, 3)
