"""Flattening of nested argument structures (reference pippy/_utils.py:13-53)."""
from __future__ import annotations

from typing import Any, List

import torch
from torch.utils import _pytree as pytree


def flatten_args(args) -> List[Any]:
    """Every leaf of a nested args structure, tensors and non-tensors alike, in traversal order."""
    leaves, _ = pytree.tree_flatten(args)
    return list(leaves)


def flatten_args_detach(args):
    """Returns ``(new_args, flat_detached)`` where every tensor leaf is detached but keeps its
    ``requires_grad`` flag, so the result starts a fresh autograd island."""
    flat_detached: List[Any] = []

    def detach(a):
        if isinstance(a, torch.Tensor):
            d = a.detach().requires_grad_(a.requires_grad)
            flat_detached.append(d)
            return d
        flat_detached.append(a)
        return a

    new_args = pytree.tree_map(detach, args)
    return new_args, flat_detached
