"""Sharded checkpoints in the HuggingFace index layout (reference pippy/utilities/hf_checkpoint.py).

Directory layout written by ``save_checkpoint`` with a world of W ranks:

    pytorch_model-{rank+1:05d}-of-{W:05d}.bin      torch.save({original_fqn: tensor}) of the rank's stage(s)
    pytorch_optim-{rank+1:05d}-of-{W:05d}.bin      torch.save(optimizer.state_dict())            (optional)
    pytorch_model.bin.index.json                   {"metadata": {"total_size": bytes},
                                                    "weight_map": {original_fqn: file name}}      (rank 0)

Keys are the ORIGINAL model's parameter names (stage modules keep them), so a checkpoint written by a pipeline of
any depth loads into any other split, or into the unsplit model.  ``load_checkpoint`` opens only the files that
hold a tensor the given module needs, materialises meta parameters on the target device and understands the usual
tied-weight aliases.
"""
from __future__ import annotations

import json
import logging
import os
import tempfile
from typing import Any, Dict, Iterable, List, Optional, Sequence, Union

import torch
import torch.distributed as dist
import torch.nn as nn

logger = logging.getLogger("pippy_b200")

CKPT_INDEX_JSON_FILENAME = "pytorch_model.bin.index.json"
DTYPE_SIZES = {
    torch.float32: 4, torch.float16: 2, torch.bfloat16: 2, torch.float64: 8, torch.int64: 8, torch.int32: 4,
    torch.int16: 2, torch.int8: 1, torch.uint8: 1, torch.bool: 1,
}
STRIP_PREFIXES = ("model.", "transformer.", "module.")
# lm-head style names and the embedding they may be tied to
TIED_ALIASES = {
    "lm_head.weight": ("wte.weight", "transformer.wte.weight", "embed_tokens.weight", "model.embed_tokens.weight",
                       "tok_embeddings.weight", "shared.weight"),
    "output.weight": ("tok_embeddings.weight",),
}


def _model_file(rank: int, world: int) -> str:
    return f"pytorch_model-{rank + 1:05d}-of-{world:05d}.bin"


def _optim_file(rank: int, world: int) -> str:
    return f"pytorch_optim-{rank + 1:05d}-of-{world:05d}.bin"


def _atomic_write(path: str, writer) -> None:
    d = os.path.dirname(path) or "."
    fd, tmp = tempfile.mkstemp(dir=d, prefix=".tmp_", suffix=os.path.basename(path))
    try:
        with os.fdopen(fd, "w") as f:
            writer(f)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def _stage_modules(stage_or_stages) -> List[nn.Module]:
    items = stage_or_stages if isinstance(stage_or_stages, (list, tuple)) else [stage_or_stages]
    mods = []
    for it in items:
        mods.append(it.submod if hasattr(it, "submod") else it)
    return mods


def _stage_state(stage_or_stages) -> Dict[str, torch.Tensor]:
    state: Dict[str, torch.Tensor] = {}
    for mod in _stage_modules(stage_or_stages):
        inner = mod.module if hasattr(mod, "module") and isinstance(mod.module, nn.Module) and \
            type(mod).__name__ == "DistributedDataParallel" else mod
        for k, v in inner.state_dict().items():
            state[k] = v.detach().cpu()
    return state


def _create_index(weight_owner: Dict[str, Dict[str, Any]], world: int) -> Dict[str, Any]:
    total = 0
    weight_map: Dict[str, str] = {}
    seen_names = set()
    for rank in range(world):
        for name, (shape, dtype) in weight_owner.get(rank, {}).items():
            weight_map.setdefault(name, _model_file(rank, world))
            if name in seen_names:
                continue  # replicated tensors count once
            seen_names.add(name)
            numel = 1
            for s in shape:
                numel *= s
            total += numel * DTYPE_SIZES.get(dtype, 4)
    return {"metadata": {"total_size": total}, "weight_map": weight_map}


def save_checkpoint(stage, checkpoint_dir: str, optimizer=None, group: Optional[dist.ProcessGroup] = None,
                    write: bool = True) -> None:
    """Every pipeline rank writes its stage(s) (``stage`` may be a list for interleaved schedules); rank 0 of
    ``group`` writes the index. With data parallelism pass ``write=(dp_rank == 0)`` so one replica writes."""
    if dist.is_initialized():
        rank, world = dist.get_rank(group), dist.get_world_size(group)
    else:
        rank, world = 0, 1
    os.makedirs(checkpoint_dir, exist_ok=True)
    state = _stage_state(stage)
    if write:
        torch.save(state, os.path.join(checkpoint_dir, _model_file(rank, world)))
        if optimizer is not None:
            torch.save(optimizer.state_dict(), os.path.join(checkpoint_dir, _optim_file(rank, world)))
    summary = {k: (tuple(v.shape), str(v.dtype)) for k, v in state.items()}
    if dist.is_initialized() and world > 1:
        gathered: List[Any] = [None] * world
        dist.all_gather_object(gathered, summary, group=group)
    else:
        gathered = [summary]
    if rank == 0 and write:
        owners = {
            r: {k: (shape, getattr(torch, dt.split(".")[-1])) for k, (shape, dt) in g.items()}
            for r, g in enumerate(gathered)
        }
        index = _create_index(owners, world)
        _atomic_write(os.path.join(checkpoint_dir, CKPT_INDEX_JSON_FILENAME),
                      lambda f: json.dump(index, f, indent=2, sort_keys=True))
    if dist.is_initialized() and world > 1:
        dist.barrier(group=group)


def _match_checkpoint_name(name: str, weight_map: Dict[str, str]) -> Optional[str]:
    if name in weight_map:
        return name
    for prefix in STRIP_PREFIXES:
        if name.startswith(prefix) and name[len(prefix):] in weight_map:
            return name[len(prefix):]
        if prefix + name in weight_map:
            return prefix + name
    leaf = name
    for head, aliases in TIED_ALIASES.items():
        if leaf.endswith(head):
            base = leaf[: -len(head)]
            for alias in aliases:
                for cand in (base + alias, alias):
                    if cand in weight_map:
                        return cand
    return None


def _set_tensor(module: nn.Module, name: str, value: torch.Tensor, device, dtype) -> None:
    """Installs ``value`` as parameter/buffer ``name``.  With ``dtype=None`` a floating-point value takes the dtype
    of the tensor it replaces (reference utilities/hf_checkpoint.py:244-324: an fp32 shard loaded into a bf16 stage
    stays bf16; integer and bool tensors are never cast).  When shape, dtype and device already match, the value is
    copied into the existing storage, so a parameter that lives in a flat buffer (``optim.FlatParams``) stays
    there; only meta tensors and genuine layout changes replace the object."""
    *path, leaf = name.split(".")
    mod = module
    for atom in path:
        mod = getattr(mod, atom)
    is_param = leaf in mod._parameters and mod._parameters[leaf] is not None
    old = mod._parameters[leaf] if is_param else mod._buffers.get(leaf)
    if value.is_floating_point():
        want = dtype if dtype is not None else (old.dtype if old is not None and old.is_floating_point() else None)
        if want is not None:
            value = value.to(want)
    if device is not None:
        value = value.to(device)
    elif old is not None and not old.is_meta:
        value = value.to(old.device)
    if is_param:
        if old.is_meta or old.shape != value.shape or old.device != value.device or old.dtype != value.dtype:
            new = nn.Parameter(value, requires_grad=old.requires_grad)
            for attr in ("main_grad",):
                if hasattr(old, attr):
                    setattr(new, attr, getattr(old, attr))
            mod._parameters[leaf] = new
        else:
            with torch.no_grad():
                old.copy_(value)
    elif leaf in mod._buffers:
        if old is None or old.is_meta or old.shape != value.shape or old.dtype != value.dtype:
            mod._buffers[leaf] = value
        else:
            old.copy_(value)
    else:
        raise KeyError(f"{name} is neither a parameter nor a buffer of the module")


def load_checkpoint(model: nn.Module, index_filename: str, optim=None, device=None, dtype=None,
                    checkpoint_prefix: Optional[str] = None, group: Optional[dist.ProcessGroup] = None,
                    strict: bool = True):
    """Loads the tensors ``model`` (a stage module, a stage, or the whole model) needs from a sharded checkpoint.
    ``checkpoint_prefix`` is prepended to the module's names when looking them up. Returns ``model``, or
    ``(model, optim)`` when an optimizer was passed (reference utilities/hf_checkpoint.py:66-146)."""
    module = model.submod if hasattr(model, "submod") else model
    with open(index_filename) as f:
        index = json.load(f)
    weight_map: Dict[str, str] = index["weight_map"]
    ckpt_dir = os.path.dirname(os.path.abspath(index_filename))
    wanted: Dict[str, List] = {}
    missing: List[str] = []
    names = [k for k in module.state_dict().keys()]
    for name in names:
        lookup = (checkpoint_prefix + name) if checkpoint_prefix else name
        found = _match_checkpoint_name(lookup, weight_map)
        if found is None:
            missing.append(name)
            continue
        wanted.setdefault(weight_map[found], []).append((name, found, found != lookup))
    if missing and strict:
        raise KeyError(f"checkpoint {index_filename} has no entry for {missing[:5]}{'...' if len(missing) > 5 else ''}")
    for fname, entries in wanted.items():
        shard = torch.load(os.path.join(ckpt_dir, fname), map_location="cpu", weights_only=True)
        for name, ckpt_name, aliased in entries:
            value = shard[ckpt_name]
            if aliased:
                value = value.clone()
            _set_tensor(module, name, value, device, dtype)
    if optim is not None:
        if dist.is_initialized():
            rank, world = dist.get_rank(group), dist.get_world_size(group)
        else:
            rank, world = 0, 1
        path = os.path.join(ckpt_dir, _optim_file(rank, world))
        if os.path.exists(path):
            optim.load_state_dict(torch.load(path, map_location="cpu", weights_only=False))
        return model, optim
    return model
