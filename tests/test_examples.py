"""The example programs run as a user would run them, on gloo ranks (reference .github/workflows/model_tests.yaml
runs its examples the same way on GPUs).  Each example checks its own result and exits non-zero on a mismatch."""
import os
import subprocess
import sys

import pytest
import torch
import torch.fx as fx

import pippy_b200 as pp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(path, nproc, *args, timeout=600):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           "--nproc-per-node", str(nproc), os.path.join(ROOT, "examples", path), *args]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res.stdout


@pytest.mark.parametrize("path,nproc", [
    ("basic/example.py", 3),
    ("basic/example_train.py", 3),
    ("basic/example_manual_stage.py", 3),
    ("mixture_of_experts/experts_as_stages.py", 5),
    ("unrolling/unroll.py", 2),
    ("cpu_init/cpu_init.py", 2),
    ("checkpoint/toy_checkpoint.py", 2),
    ("profiling/mlp_profiling.py", 2),
    ("huggingface/pippy_unet.py", 2),
])
def test_example_runs(path, nproc, tmp_path):
    _run(path, nproc)


@pytest.mark.parametrize("nproc", [2, 4])
def test_llama_greedy_decoding_same_tokens_as_unsplit_model(nproc):
    """Hugging Face Llama through the traced pipeline, greedy decoding of several tokens: the same tokens on 2 and
    4 ranks as the unsplit model chooses (reference examples/llama/README.md:1-17 expects the same words on 2, 4, 8)."""
    out = _run("llama/pippy_llama.py", nproc, "--check", "--new-tokens", "3", "--cuda", "0")
    assert "chose the same 3 token(s)" in out


def test_parallel_branches_keep_stage_order():
    """Stages that read the same producer side by side: stage i must be submod_i in the program text and in
    the runtime's topology (fx.split_module emits such branches in an order of its own)."""
    sys.path.insert(0, os.path.join(ROOT, "examples", "mixture_of_experts"))
    from experts_as_stages import D_HID, ExpertsSideBySide

    torch.manual_seed(0)
    model = ExpertsSideBySide(3)
    x = torch.randn(4, D_HID)
    split = {"pre_proc": pp.SplitPoint.END, **{f"experts.{i}": pp.SplitPoint.END for i in range(3)}}
    pipe = pp.pipeline(model, 1, example_args=(x,), split_spec=split)
    calls = [str(n.target) for n in pipe.split_gm.graph.nodes if n.op == "call_module"]
    assert calls == [f"submod_{i}" for i in range(5)]
    stage = pp.PipelineStage(pipe, 4, torch.device("cpu"))
    assert [s.source for s in stage.input_specs] == [1, 2, 3]
    first = pp.PipelineStage(pipe, 0, torch.device("cpu"))
    assert first.output_dests[0] == [1, 2, 3]
