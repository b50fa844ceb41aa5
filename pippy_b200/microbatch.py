"""Microbatch split and merge (reference: pippy/microbatch.py).

``split_args_kwargs_into_chunks`` turns full-batch ``(args, kwargs)`` into per-microbatch lists;
``merge_chunks`` is its inverse for stage outputs.  Chunking is described per leaf by a
:class:`TensorChunkSpec` (split this dimension), :class:`_Replicate` (same value in every microbatch)
or, for merging only, a :class:`_CustomReducer` (fold the per-microbatch values).
"""
from __future__ import annotations

import logging
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
from torch.utils import _pytree as pytree

logger = logging.getLogger("pippy_b200")

# When True every "chunk" is a full-size tensor that is zero outside its own slice, so a row-independent
# model produces bit-identical rows to the full-batch run (reference microbatch.py:16, 143-163).
_debug_mask_minibatches = False

DEFAULT_CHUNK_DIM = 0


class _CustomReducer:
    """Merge rule for a value that is folded rather than concatenated, e.g. a scalar loss."""

    def __init__(self, init_value, reduce_fn: Callable[[Any, Any], Any]):
        self.init_value = init_value
        self.reduce_fn = reduce_fn


class _LossReducer(_CustomReducer):
    pass


sum_reducer = _LossReducer(torch.tensor(0.0), lambda a, b: a + b)


class TensorChunkSpec:
    """Marks a tensor leaf as split along ``split_dim`` (reference microbatch.py:44-63)."""

    def __init__(self, split_dim: int):
        self.split_dim = split_dim

    split_dim: int

    def __repr__(self) -> str:
        return f"{self.__class__.__module__}.{self.__class__.__name__}({self.split_dim})"

    def __str__(self) -> str:
        return f"TensorChunkSpec({self.split_dim})"

    def __eq__(self, other) -> bool:
        return isinstance(other, TensorChunkSpec) and other.split_dim == self.split_dim

    def __hash__(self) -> int:
        return hash(("TensorChunkSpec", self.split_dim))


class _Replicate:
    """Marks a leaf as identical in every microbatch."""


def _mask_chunks(v: torch.Tensor, pieces: Sequence[torch.Tensor], dim: int) -> List[torch.Tensor]:
    out = []
    start = 0
    for piece in pieces:
        size = piece.size(dim)
        masked = torch.zeros_like(v)
        index = [slice(None)] * v.dim()
        index[dim] = slice(start, start + size)
        masked[tuple(index)] = v[tuple(index)]
        out.append(masked)
        start += size
    return out


def _shard_leaves(values: Dict[Any, Any], specs: Dict[Any, Any], chunks: int, what: str) -> List[Dict[Any, Any]]:
    """Chunks every entry of ``values`` (a dict keyed by position or name) according to ``specs``.

    Returns one dict per chunk. The chunk count may shrink if the first tensor is shorter than
    ``chunks`` along its split dimension (reference microbatch.py:120-137).
    """
    flat_per_key: Dict[Any, Tuple[List[List[Any]], Any]] = {}
    real_chunks = chunks
    first_tensor = True
    for key, value in values.items():
        leaves, tree = pytree.tree_flatten(value)
        spec = specs[key]
        spec_leaves, _ = pytree.tree_flatten(spec, is_leaf=lambda s: isinstance(s, (TensorChunkSpec, _Replicate)))
        if len(leaves) != len(spec_leaves):
            raise ValueError(
                f"{what} {key!r} did not have the same number of values as chunk spec: "
                f"{len(leaves)} values vs {len(spec_leaves)} spec entries"
            )
        per_leaf: List[List[Any]] = []
        for leaf, leaf_spec in zip(leaves, spec_leaves):
            if leaf_spec is _Replicate or isinstance(leaf_spec, _Replicate) or not isinstance(leaf, torch.Tensor):
                per_leaf.append([leaf] * real_chunks)
                continue
            if not isinstance(leaf_spec, TensorChunkSpec):
                raise TypeError(f"Unrecognized chunk spec: {leaf_spec}")
            dim = leaf_spec.split_dim
            extent = leaf.size(dim)
            if extent < real_chunks:
                if first_tensor:
                    logger.warning(
                        "Tensor size on chunking dimension is %d, downsizing the number of chunks from %d to %d.",
                        extent, real_chunks, extent,
                    )
                    real_chunks = extent
                else:
                    raise RuntimeError(
                        f"{what} {key!r} has {extent} elements on chunking dimension {dim}, fewer than the "
                        f"{real_chunks} chunks established by an earlier tensor"
                    )
            first_tensor = False
            pieces = list(torch.tensor_split(leaf, real_chunks, dim))
            if _debug_mask_minibatches:
                pieces = _mask_chunks(leaf, pieces, dim)
            per_leaf.append(pieces)
        flat_per_key[key] = (per_leaf, tree)

    result: List[Dict[Any, Any]] = []
    for c in range(real_chunks):
        entry = {}
        for key, (per_leaf, tree) in flat_per_key.items():
            # leaves replicated before a downsize happened may be longer than real_chunks; index is still valid
            entry[key] = pytree.tree_unflatten([leaf_chunks[c] for leaf_chunks in per_leaf], tree)
        result.append(entry)
    return result


def split_args_kwargs_into_chunks(
    args: Tuple[Any, ...],
    kwargs: Optional[Dict[str, Any]],
    chunks: int,
    args_chunk_spec: Optional[Tuple[Any, ...]] = None,
    kwargs_chunk_spec: Optional[Dict[str, Any]] = None,
) -> Tuple[List[Tuple], List[Dict]]:
    """Splits positional and keyword arguments into ``chunks`` microbatches.

    By default every tensor is split along dimension 0 with ``torch.tensor_split`` (uneven sizes allowed) and
    every non-tensor is replicated. A chunk spec mirrors the structure of the value it describes.
    Returns ``(args_per_chunk, kwargs_per_chunk)``; both lists have the same length, which can be smaller
    than ``chunks`` when the batch is shorter than the requested count.
    """
    kwargs = {} if kwargs is None else kwargs
    args = tuple(args)

    def default_spec(value):
        return pytree.tree_map(lambda _: TensorChunkSpec(DEFAULT_CHUNK_DIM), value)

    if args_chunk_spec is None:
        args_chunk_spec = tuple(default_spec(a) for a in args)
    if kwargs_chunk_spec is None:
        kwargs_chunk_spec = {k: default_spec(v) for k, v in kwargs.items()}
    if len(args_chunk_spec) != len(args):
        raise ValueError(
            f"args did not have the same number of values as chunk spec: {len(args)} vs {len(args_chunk_spec)}"
        )
    if set(kwargs_chunk_spec.keys()) != set(kwargs.keys()):
        raise ValueError(
            f"kwargs did not have the same number of values as chunk spec: {sorted(kwargs)} vs "
            f"{sorted(kwargs_chunk_spec)}"
        )

    arg_values = dict(enumerate(args))
    arg_specs = dict(enumerate(args_chunk_spec))
    args_split = _shard_leaves(arg_values, arg_specs, chunks, "argument")
    real_chunks = len(args_split) if args else chunks
    kwargs_split = _shard_leaves(kwargs, kwargs_chunk_spec, real_chunks, "keyword argument")
    if kwargs and len(kwargs_split) < real_chunks:
        # keyword tensors forced a smaller count: redo the positional split with it
        real_chunks = len(kwargs_split)
        args_split = _shard_leaves(arg_values, arg_specs, real_chunks, "argument")
    if args and kwargs and len(args_split) != len(kwargs_split):
        raise RuntimeError(
            f"args and kwargs were split into different numbers of chunks: {len(args_split)} vs {len(kwargs_split)}"
        )
    if not args:
        args_split = [{} for _ in range(len(kwargs_split) if kwargs else real_chunks)]
    if not kwargs:
        kwargs_split = [{} for _ in range(len(args_split))]

    args_out = [tuple(chunk[i] for i in range(len(args))) for chunk in args_split]
    return args_out, kwargs_split


def merge_chunks(chunks: List[Any], chunk_spec=None):
    """Rebuilds a full-batch value from per-microbatch values (reference microbatch.py:303-432).

    ``chunk_spec`` mirrors one chunk's structure. ``None`` means "concatenate every tensor along dim 0".
    ``TensorChunkSpec`` leaves are concatenated, ``_CustomReducer`` leaves folded, any other leaf must be equal in
    every chunk and the first one is returned.
    """
    if len(chunks) == 0:
        raise ValueError("merge_chunks needs at least one chunk")
    leaves0, tree = pytree.tree_flatten(chunks[0])
    if chunk_spec is None:
        spec_leaves: List[Any] = [
            TensorChunkSpec(DEFAULT_CHUNK_DIM) if isinstance(leaf, torch.Tensor) else None for leaf in leaves0
        ]
    else:
        spec_leaves, _ = pytree.tree_flatten(
            chunk_spec, is_leaf=lambda s: isinstance(s, (TensorChunkSpec, _Replicate, _CustomReducer))
        )
        if len(spec_leaves) != len(leaves0):
            raise ValueError(
                f"chunk spec has {len(spec_leaves)} entries but the chunks have {len(leaves0)} values"
            )
    per_chunk_leaves = []
    for chunk in chunks:
        leaves, _ = pytree.tree_flatten(chunk)
        if len(leaves) != len(leaves0):
            raise ValueError("chunks do not all have the same structure")
        per_chunk_leaves.append(leaves)

    merged = []
    for idx, spec in enumerate(spec_leaves):
        values = [leaves[idx] for leaves in per_chunk_leaves]
        if isinstance(spec, TensorChunkSpec):
            if _debug_mask_minibatches:
                # every value is full size; take each chunk's own slice back out
                dim = spec.split_dim
                meta = torch.empty(values[0].shape, device="meta")
                bounds = [0]
                for piece in torch.tensor_split(meta, len(values), dim):
                    bounds.append(bounds[-1] + piece.size(dim))
                sliced = []
                for c, v in enumerate(values):
                    index = [slice(None)] * v.dim()
                    index[dim] = slice(bounds[c], bounds[c + 1])
                    sliced.append(v[tuple(index)])
                values = sliced
            if all(isinstance(v, torch.Tensor) and v.dim() == 0 for v in values):
                merged.append(torch.stack(values))
            else:
                merged.append(torch.cat(values, dim=spec.split_dim))
        elif isinstance(spec, _CustomReducer):
            acc = spec.init_value
            for v in values:
                acc = spec.reduce_fn(acc, v)
            merged.append(acc)
        else:
            first = values[0]
            for v in values[1:]:
                same = torch.equal(first, v) if isinstance(first, torch.Tensor) and isinstance(v, torch.Tensor) else first == v
                if not same:
                    raise AssertionError(f"value {idx} is marked as replicated but differs between chunks")
            merged.append(first)
    return pytree.tree_unflatten(merged, tree)
