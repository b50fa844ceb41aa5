"""Tracing front-end, single process (reference test/test_pipe.py, test_unflatten.py, test_transformer.py,
test_chunkspec.py, test_pipe_bwd.py, test_autosplit.py and the still-relevant parts of test_ir.py)."""
import copy
import pickle

import pytest
import torch
import torch.nn as nn

from pippy_b200.ir import (
    ArgsChunkSpec, KwargsChunkSpec, MultiUseParameterConfig, Pipe, PipeSequential, SplitPoint, TrivialLossWrapper,
    annotate_split_points, pipe_split, pipeline,
)
from pippy_b200.split_policies import split_by_graph, split_into_equal_size, split_on_size_threshold

D = 32


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(4, 4, 3, padding=1)
        self.lin = nn.Linear(D, D)
        self.register_buffer("scale", torch.full((D,), 0.5))

    def forward(self, x, extra=None):
        y = self.lin(x) * self.scale
        pipe_split()
        y = torch.relu(y)
        y.add_(1.0)  # in-place op inside a stage
        return y if extra is None else y + extra


class Model(nn.Module):
    def __init__(self):
        super().__init__()
        self.block0, self.block1 = Block(), Block()
        self.head = nn.Linear(D, 8)

    def forward(self, x, y=torch.zeros(4, D)):
        x = self.block0(x, y)
        pipe_split()
        x = self.block1(x)
        return self.head(x)


def _union_keys(pipe):
    keys = set()
    for i in range(pipe.num_stages):
        keys |= set(pipe.get_stage_module(i).state_dict().keys())
    return keys


def test_nested_splits_output_and_state_dict_keys():
    torch.manual_seed(0)
    mod = Model()
    x, y = torch.randn(8, D), torch.randn(8, D)
    ref = mod(x, y)
    pipe = pipeline(mod, 2, (x,), {"y": y})
    assert pipe.num_stages == 4
    torch.testing.assert_close(pipe(x, y=y)[0], ref)
    torch.testing.assert_close(pipe(x, y)[0], ref)
    used = {k for k in mod.state_dict() if "conv" not in k}  # conv is never called, so no stage owns it
    assert _union_keys(pipe) == used
    for i in range(pipe.num_stages):
        for k in pipe.get_stage_module(i).state_dict():
            assert k in mod.state_dict()
    # buffers stay buffers, parameters stay parameters
    sub = pipe.get_stage_module(0)
    assert "block0.scale" in dict(sub.named_buffers()) and "block0.lin.weight" in dict(sub.named_parameters())
    assert pipe.info().num_chunks == 2
    with pytest.raises(ValueError, match="Invalid stage index"):
        pipe.get_stage_module(4)
    with pytest.raises(RuntimeError, match="invoke the Pipe object directly"):
        pipe.split_gm(x)


def test_argument_binding_errors():
    mod = Model()
    x, y = torch.randn(8, D), torch.randn(8, D)
    pipe = pipeline(mod, 2, (x,), {"y": y})
    with pytest.raises(TypeError, match="unexpected keyword argument 'z'"):
        pipe(x, z=y)
    with pytest.raises(TypeError, match="multiple values for argument 'y'"):
        pipe(x, y, y=y)


class Layer(nn.Module):
    def __init__(self):
        super().__init__()
        self.w1, self.w2 = nn.Linear(D, D), nn.Linear(D, D)

    def forward(self, x):
        return x + self.w2(torch.relu(self.w1(x)))


class Transformer(nn.Module):
    def __init__(self, n=8):
        super().__init__()
        self.layers = nn.ModuleList([Layer() for _ in range(n)])
        self.out = nn.Linear(D, 4)

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return self.out(x)


def test_split_spec_beginning_and_end_and_errors():
    mod = Transformer()
    x = torch.randn(4, D)
    ref = mod(x)
    pipe = pipeline(copy.deepcopy(mod), 2, (x,), split_spec={"layers.4": SplitPoint.BEGINNING})
    assert pipe.num_stages == 2
    torch.testing.assert_close(pipe(x)[0], ref)
    s0 = {k.split(".")[1] for k in pipe.get_stage_module(0).state_dict() if k.startswith("layers.")}
    s1 = {k.split(".")[1] for k in pipe.get_stage_module(1).state_dict() if k.startswith("layers.")}
    assert s0 == {"0", "1", "2", "3"} and s1 == {"4", "5", "6", "7"}
    pipe = pipeline(copy.deepcopy(mod), 2, (x,), split_spec={"layers.1": SplitPoint.END, "layers.5": SplitPoint.END})
    assert pipe.num_stages == 3
    torch.testing.assert_close(pipe(x)[0], ref)
    with pytest.raises(AttributeError, match="Specified target layers.9.w1 referenced nonexistent module layers.9"):
        annotate_split_points(copy.deepcopy(mod), {"layers.9.w1": SplitPoint.END})
    with pytest.raises(ValueError, match="Unknown split point type"):
        annotate_split_points(copy.deepcopy(mod), {"layers.1": "end"})
    with pytest.raises(ValueError, match="Cannot specify both"):
        pipeline(copy.deepcopy(mod), 2, (x,), split_spec={"layers.1": SplitPoint.END}, split_policy=split_into_equal_size(2))


def test_consecutive_and_trailing_markers_collapse():
    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = nn.Linear(D, D), nn.Linear(D, D)

        def forward(self, x):
            pipe_split()
            x = self.a(x)
            pipe_split()
            pipe_split()
            x = self.b(x)
            pipe_split()
            return x

    x = torch.randn(4, D)
    mod = M()
    pipe = pipeline(mod, 2, (x,))
    assert pipe.num_stages == 2
    torch.testing.assert_close(pipe(x)[0], mod(x))


def test_newer_call_style_and_build_stage_info():
    mod = Transformer(4)
    x_mb = torch.randn(2, D)
    pipe = pipeline(mod, mb_args=(x_mb,), split_spec={"layers.2": SplitPoint.BEGINNING})
    assert pipe.num_stages == 2 and pipe.info().num_chunks is None
    torch.testing.assert_close(pipe(x_mb)[0], mod(x_mb))


def test_chunk_spec_context_managers():
    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(D, D)

        def forward(self, x, y, z=None):
            x = self.lin(x)
            pipe_split()
            return x + y + z

    x, y, z = torch.randn(6, D), torch.randn(6, D), torch.randn(6, D)
    with ArgsChunkSpec((0, 0)), KwargsChunkSpec({"z": 0}):
        pipe = pipeline(M(), 3, (x, y), {"z": z})
    info = pipe.info()
    assert info.args_chunk_spec is not None and info.kwargs_chunk_spec is not None
    assert Pipe.args_chunk_spec is None and Pipe.kwargs_chunk_spec is None
    assert pipe.num_stages == 2


class Tied(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(16, D)
        self.mid = nn.Linear(D, D)
        self.head = nn.Linear(D, 16, bias=False)
        self.head.weight = self.emb.weight

    def forward(self, ids):
        x = self.emb(ids)
        pipe_split()
        x = self.mid(x)
        pipe_split()
        return self.head(x)


def test_tied_weights_replicate_and_transmit():
    torch.manual_seed(0)
    mod = Tied()
    ids = torch.randint(0, 16, (4, 5))
    ref = mod(ids)
    pipe = pipeline(copy.deepcopy(mod), 2, (ids,))
    assert pipe.num_stages == 3
    assert pipe.replicated_params == [{"submod_0": "emb.weight", "submod_2": "emb.weight"}]
    w0 = pipe.get_stage_module(0).emb.weight
    w2 = pipe.get_stage_module(2).head.weight
    assert w0 is not w2 and torch.equal(w0, w2)
    assert pipe.get_stage_module(2).emb.weight is w2  # both original names exist and alias inside the stage
    torch.testing.assert_close(pipe(ids)[0], ref)
    assert _union_keys(pipe) == set(mod.state_dict().keys())

    pipe_t = pipeline(copy.deepcopy(mod), 2, (ids,), multi_use_param_spec=MultiUseParameterConfig.TRANSMIT)
    assert pipe_t.replicated_params == []
    assert "emb.weight" not in pipe_t.get_stage_module(2).state_dict()
    torch.testing.assert_close(pipe_t(ids)[0], ref)
    with pytest.raises(ValueError, match="Unknown multi-use config"):
        pipeline(copy.deepcopy(mod), 2, (ids,), multi_use_param_spec={"emb.weight": "nope"})


def test_loss_in_forward_generates_backward():
    torch.manual_seed(0)
    base = PipeSequential.from_sequential(nn.Sequential(nn.Linear(D, D), nn.ReLU(), nn.Linear(D, D), nn.Linear(D, 4)))
    wrapper = TrivialLossWrapper(base, nn.MSELoss(reduction="sum"))
    ref = copy.deepcopy(wrapper)
    x, t = torch.randn(8, D), torch.randn(8, 4)
    pipe = pipeline(wrapper, 2, (x, t))
    assert pipe.has_loss_and_backward and pipe.num_stages == 4
    assert any(n.op == "call_function" and n.target.__name__ == "stage_backward" for n in pipe.split_gm.graph.nodes)
    loss = pipe(x, t)[0]
    ref_loss = ref(x, t)
    ref_loss.backward()
    torch.testing.assert_close(loss, ref_loss)
    ref_grads = {k: p.grad for k, p in ref.named_parameters()}
    for i in range(pipe.num_stages):
        for k, p in pipe.get_stage_module(i).named_parameters():
            torch.testing.assert_close(p.grad, ref_grads[k], msg=k)


def test_auto_split_policies():
    mod = Transformer(8)
    x = torch.randn(4, D)
    ref = mod(x)
    for n in (2, 4):
        pipe = pipeline(copy.deepcopy(mod), 2, (x,), split_policy=split_into_equal_size(n))
        assert pipe.num_stages == n
        torch.testing.assert_close(pipe(x)[0], ref)
        sizes = [sum(p.numel() for p in pipe.get_stage_module(i).parameters()) for i in range(n)]
        assert max(sizes) <= 2 * (sum(sizes) / n)
    per_layer = 2 * (D * D + D)
    pipe = pipeline(copy.deepcopy(mod), 2, (x,), split_policy=split_on_size_threshold(2 * per_layer))
    assert pipe.num_stages >= 4
    torch.testing.assert_close(pipe(x)[0], ref)
    assert _union_keys(pipe) == set(mod.state_dict().keys())


def test_graph_split_policy():
    pytest.importorskip("scipy")
    mod = Transformer(6)
    x = torch.randn(4, D)
    pipe = pipeline(copy.deepcopy(mod), 2, (x,), split_policy=split_by_graph(3))
    assert pipe.num_stages == 3
    torch.testing.assert_close(pipe(x)[0], mod(x))
    sizes = [sum(p.numel() for p in pipe.get_stage_module(i).parameters()) for i in range(3)]
    assert max(sizes) <= 2.5 * sum(sizes) / 3 + 1


def test_device_rewrite_of_traced_factory_ops():
    from pippy_b200.utils.graph import modify_graph_op_device

    class M(nn.Module):
        def forward(self, x):
            return x + torch.ones(x.shape[-1], device=x.device)

    pipe = pipeline(M(), 1, (torch.randn(2, 4),))
    sub = pipe.get_stage_module(0)
    modify_graph_op_device(sub, torch.device("meta"))
    devs = [n.kwargs["device"] for n in sub.graph.nodes if n.op == "call_function" and "device" in n.kwargs]
    assert devs and all(d == torch.device("meta") for d in devs)


def test_stage_module_pickles_by_node_list():
    from pippy_b200.serialization import enable_direct_serialization

    class Long(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(D, D)

        def forward(self, x):
            x = self.lin(x)
            for _ in range(300):
                x = x + 1.0
            return x

    pipe = pipeline(Long(), 1, (torch.randn(2, D),))
    sub = enable_direct_serialization(pipe.get_stage_module(0))
    clone = pickle.loads(pickle.dumps(sub))
    x = torch.randn(2, D)
    torch.testing.assert_close(clone(x), sub(x))


def test_remap_qualname():
    pipe = pipeline(Transformer(4), 2, (torch.randn(4, D),), split_spec={"layers.2": SplitPoint.BEGINNING})
    assert pipe.remap_qualname("split_gm.submod_1.layers.2.w1.weight") == "layers.2.w1.weight"
    assert pipe.remap_qualname("submod_0.layers.0.w2.bias") == "layers.0.w2.bias"
