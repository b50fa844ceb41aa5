"""Package logging and compact rendering of values in error messages.

The log level comes from the environment variable ``PIPPY_VERBOSITY`` (WARNING, INFO or DEBUG), read once at
import, as in the reference (pippy/_debug.py:8-21); unlike the reference nothing is logged when the variable
is unset.
"""
from __future__ import annotations

import logging
import os

import torch

logger = logging.getLogger("pippy_b200")

_LEVELS = {"WARNING": logging.WARNING, "INFO": logging.INFO, "DEBUG": logging.DEBUG}


def _configure() -> None:
    raw = os.environ.get("PIPPY_VERBOSITY")
    if raw is None:
        return
    level = _LEVELS.get(raw.upper())
    if level is None:
        logger.setLevel(logging.WARNING)
        logger.warning("Unsupported PIPPY_VERBOSITY level %r; using WARNING", raw)
        return
    logger.setLevel(level)
    if not logger.handlers and not logging.getLogger().handlers:
        logging.basicConfig(format="%(asctime)s %(name)s %(levelname)s %(message)s")


_configure()


def friendly_debug_info(v) -> str:
    """``Tensor(shape, grad=..., dtype=...)`` for tensors, ``str`` for everything else."""
    if isinstance(v, torch.Tensor):
        return f"Tensor({tuple(v.shape)}, grad={v.requires_grad}, dtype={v.dtype})"
    return str(v)


def map_debug_info(a):
    """Applies :func:`friendly_debug_info` to every leaf of a nested args structure (pippy/_debug.py:33-39)."""
    from torch.utils import _pytree as pytree

    return pytree.tree_map(friendly_debug_info, a)
