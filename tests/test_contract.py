"""Error conditions and messages a user of the reference relies on (the reference raises them at pippy/_IR.py:653-656,
602-607, 1324-1338, 1373-1376; _PipelineStage.py:99-117, 472-484; ManualPipelineStage.py:144-175;
PipelineSchedule.py:466-469; _debug.py:13-18)."""
import importlib
import logging

import pytest
import torch
import torch.nn as nn

import pippy_b200 as pp
from pippy_b200.manual_stage import get_stage_shapes


class M(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4))
        self.b = nn.Linear(4, 4)

    def forward(self, x):
        return self.b(self.a(x))


def test_pipeline_argument_errors():
    x = torch.randn(4, 4)
    with pytest.raises(ValueError, match="Cannot specify both `split_spec` and `split_policy`"):
        pp.pipeline(M(), 2, (x,), split_spec={"a": pp.SplitPoint.END}, split_policy=pp.split_into_equal_size(2))
    with pytest.raises(AttributeError, match="Specified target a.zz.c referenced nonexistent module a.zz"):
        pp.annotate_split_points(M(), {"a.zz.c": pp.SplitPoint.END})
    with pytest.raises(AttributeError, match="referenced nonexistent module q$"):
        pp.annotate_split_points(M(), {"q.zz.c": pp.SplitPoint.END})
    with pytest.raises(ValueError, match="Unknown split point type."):
        pp.annotate_split_points(M(), {"a": "END"})


def test_pipe_object_errors():
    x = torch.randn(4, 4)
    pipe = pp.pipeline(M(), 2, (x,), split_spec={"a": pp.SplitPoint.END})
    assert pipe.num_stages == 2
    assert [n for n, _ in pipe.split_gm.named_children()] == ["submod_0", "submod_1"]
    with pytest.raises(ValueError, match="Invalid stage index 5!"):
        pipe.get_stage_module(5)
    with pytest.raises(RuntimeError, match="invoke the Pipe object directly, not `split_gm`"):
        pipe.split_gm(x)
    assert pipe.info().num_stages == 2 and pipe.info().num_chunks == 2


def test_stage_and_schedule_constructor_errors():
    lin = nn.Linear(4, 4)
    with pytest.raises(ValueError, match="out of range"):
        pp.ManualPipelineStage(lin, 3, 2, torch.device("cpu"), 2, input_args=torch.empty(2, 4))
    one = pp.ManualPipelineStage(lin, 0, 1, torch.device("cpu"), 2, input_args=torch.empty(2, 4))
    with pytest.raises(ValueError, match="at least 2 stages per rank"):
        pp.ScheduleInterleaved1F1B([one], 2)
    with pytest.raises(ValueError, match="at least 2 stages per rank"):
        pp.ScheduleLoopedBFS([one], 2)
    with pytest.raises(RuntimeError, match="Microbatch is required for first stage"):
        get_stage_shapes([lin], [0], 1, 0, 1, torch.device("cpu"))


def test_forward_failure_names_the_argument_shapes():
    class Bad(nn.Module):
        def forward(self, x):
            return x @ torch.randn(7, 7)

    st = pp.ManualPipelineStage(Bad(), 0, 1, torch.device("cpu"), 1, input_args=torch.empty(2, 4),
                                output_args=torch.empty(2, 4))
    with pytest.raises(RuntimeError, match=r"failed to run forward:\s+args: \['Tensor\(\(2, 4\)"):
        pp.ScheduleGPipe(st, 1).step(torch.randn(2, 4))


def test_meta_parameters_are_left_for_the_user_to_materialise():
    meta = nn.Linear(4, 4, device="meta")
    st = pp.ManualPipelineStage(meta, 0, 1, torch.device("cpu"), 1, input_args=torch.empty(2, 4, device="meta"))
    assert all(p.is_meta for p in st.submod.parameters())
    assert [tuple(m.shape) for m in st.output_metas] == [(2, 4)]


def test_verbosity_environment_variable(monkeypatch, capsys):
    import pippy_b200._debug as dbg

    monkeypatch.setenv("PIPPY_VERBOSITY", "DEBUG")
    importlib.reload(dbg)
    assert dbg.logger.level == logging.DEBUG
    monkeypatch.setenv("PIPPY_VERBOSITY", "LOUD")
    importlib.reload(dbg)
    assert dbg.logger.level == logging.WARNING
    monkeypatch.delenv("PIPPY_VERBOSITY")
    importlib.reload(dbg)
