"""Microbatch split/merge contract (reference test/test_microbatch.py, test/test_ir.py:583-775)."""
import pytest
import torch

import pippy_b200.microbatch as mb
from pippy_b200.microbatch import (
    TensorChunkSpec, _CustomReducer, _Replicate, merge_chunks, split_args_kwargs_into_chunks, sum_reducer,
)


def test_split_default_dim0_and_merge_roundtrip():
    x0, x1 = torch.randn(128, 4), torch.randn(128, 8)
    args, kwargs = split_args_kwargs_into_chunks((x0,), {"k": x1}, 4)
    assert len(args) == len(kwargs) == 4
    assert args[0][0].shape == (32, 4) and kwargs[3]["k"].shape == (32, 8)
    merged = merge_chunks([a[0] for a in args], TensorChunkSpec(0))
    torch.testing.assert_close(merged, x0)
    merged_kw = merge_chunks(kwargs, {"k": TensorChunkSpec(0)})
    torch.testing.assert_close(merged_kw["k"], x1)


def test_uneven_and_nondefault_dim_and_replicate():
    x = torch.randn(10, 6)
    args, _ = split_args_kwargs_into_chunks((x, 7, x), None, 3, (TensorChunkSpec(1), _Replicate(), _Replicate()))
    assert [a[0].shape[1] for a in args] == [2, 2, 2]
    assert all(a[1] == 7 and a[2] is x for a in args)
    args, _ = split_args_kwargs_into_chunks((torch.randn(10, 3),), None, 4)
    assert [a[0].shape[0] for a in args] == [3, 3, 2, 2]


def test_nested_structures():
    a, b = torch.randn(8, 2), torch.randn(8, 5)
    args, kwargs = split_args_kwargs_into_chunks(((a, {"b": b}),), None, 2)
    assert args[1][0][0].shape == (4, 2) and args[1][0][1]["b"].shape == (4, 5)


def test_downsize_on_first_tensor_and_error_later():
    args, _ = split_args_kwargs_into_chunks((torch.randn(2, 3),), None, 4)
    assert len(args) == 2
    with pytest.raises(RuntimeError):
        split_args_kwargs_into_chunks((torch.randn(8, 3), torch.randn(2, 3)), None, 4)


def test_spec_errors():
    with pytest.raises(ValueError, match="same number of values as chunk spec"):
        split_args_kwargs_into_chunks(((torch.randn(4), torch.randn(4)),), None, 2, ((TensorChunkSpec(0),),))
    with pytest.raises(TypeError, match="Unrecognized chunk spec"):
        split_args_kwargs_into_chunks((torch.randn(4),), None, 2, ("bogus",))


def test_custom_reducer_and_replicated_merge():
    chunks = [(torch.tensor(1.0), torch.ones(2, 3), 5), (torch.tensor(2.0), torch.ones(2, 3), 5)]
    out = merge_chunks(chunks, (sum_reducer, TensorChunkSpec(0), None))
    assert out[0].item() == 3.0 and out[1].shape == (4, 3) and out[2] == 5
    with pytest.raises(AssertionError):
        merge_chunks([(1,), (2,)], (None,))
    r = _CustomReducer(torch.tensor(0.0), lambda a, b: torch.maximum(a, b))
    assert merge_chunks([torch.tensor(1.0), torch.tensor(4.0)], r).item() == 4.0


def test_mask_mode_is_bit_exact():
    x = torch.randn(8, 4)
    lin = torch.nn.Linear(4, 4)
    try:
        mb._debug_mask_minibatches = True
        args, _ = split_args_kwargs_into_chunks((x,), None, 4)
        assert all(a[0].shape == x.shape for a in args)
        outs = [lin(a[0]) for a in args]
        merged = merge_chunks(outs, TensorChunkSpec(0))
    finally:
        mb._debug_mask_minibatches = False
    assert torch.equal(merged, lin(x))
