"""Hugging Face families through the tracing front-end (reference test/hf_test.py and examples/huggingface/*).

Each family is built tiny and random-initialised, cut into two stages at the middle block, and the Pipe's
single-process execution is compared with the unsplit model.  One family also runs across two gloo ranks.
"""
import os
import subprocess
import sys

import pytest
import torch
import torch.utils._pytree as pytree

transformers = pytest.importorskip("transformers")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "examples", "huggingface"))
import hf_utils  # noqa: E402

import pippy_b200 as pp  # noqa: E402


def _tensors(tree):
    if hasattr(tree, "to_tuple"):
        tree = tree.to_tuple()
    return [x for x in pytree.tree_leaves(tree) if isinstance(x, torch.Tensor)]


@pytest.mark.parametrize("name", sorted(hf_utils.FAMILIES))
def test_family_splits_and_matches(name):
    torch.manual_seed(0)
    model, config, fam = hf_utils.build_model(name)
    args, kwargs = hf_utils.generate_inputs(name, config, batch=4)
    pipe = pp.pipeline(model, 2, example_args=args, example_kwargs=kwargs,
                       split_spec=hf_utils.equal_layer_split(name, config, 2))
    assert pipe.num_stages == 2
    # Every parameter keeps its original fully qualified name in exactly the stages that use it.
    original = {n for n, _ in model.named_parameters(remove_duplicate=False)}
    staged = set()
    for i in range(pipe.num_stages):
        staged |= set(dict(pipe.get_stage_module(i).named_parameters()).keys())
    assert staged <= original
    mb_args = tuple(a[:2] for a in args)
    mb_kwargs = {k: v[:2] for k, v in kwargs.items()}
    with torch.no_grad():
        got, want = _tensors(pipe(*mb_args, **mb_kwargs)), _tensors(model(*mb_args, **mb_kwargs))
    assert len(got) == len(want) >= 1
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)


def test_equal_layer_split_rejects_too_many_stages():
    _, config, _ = hf_utils.build_model("gpt2")
    with pytest.raises(ValueError):
        hf_utils.equal_layer_split("gpt2", config, 5)


def test_gpt2_example_runs_on_two_ranks():
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           "--nproc-per-node", "2", os.path.join(ROOT, "examples", "huggingface", "pippy_hf.py"), "--model", "gpt2"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "pipeline output equals the unsplit model" in res.stdout


@pytest.mark.parametrize("name", sorted(hf_utils.FAMILIES))
def test_family_trains_through_traced_stages(name):
    """Every registered family (reference test/hf_test.py:796-1101 parametrises forward + backward over the model
    zoo the same way): forward + backward under 1F1B on two gloo ranks, loss and every parameter gradient equal the
    unsplit model's; weights tied across stages are replicated and their gradients sum (GPT-2, BERT), encoder
    outputs skip over the stage boundary into every decoder layer (mBART, Blenderbot), a float mask that crosses the
    boundary without a gradient gets zeros sent back (DeBERTa)."""
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
           "--nproc-per-node", "2", os.path.join(ROOT, "examples", "huggingface", "pippy_hf.py"), "--model", name,
           "--train"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    assert "parameter gradients" in res.stdout
