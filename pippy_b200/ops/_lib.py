"""ctypes binding to the in-tree CUDA library ``pippy_b200/lib/libpippy_b200.so``.

Every CUDA op of the package goes through :func:`lib`.  On a machine with a GPU a missing or
unloadable library is a hard error (there is no eager fallback for CUDA tensors); on a CPU-only
machine the library is simply not needed because CPU tensors take the plain PyTorch path.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_LIB = None
_LOCK = threading.Lock()
_ERR_WORDS: dict[int, torch.Tensor] = {}

_LIB_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib")
# PIPPY_BOUNDS_CHECK=1 selects the debug library, whose kernels validate the indices they read from tensors
LIB_PATH = os.path.join(_LIB_DIR, "libpippy_b200_dbg.so" if os.environ.get("PIPPY_BOUNDS_CHECK", "0") == "1"
                        else "libpippy_b200.so")

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


class KernelError(RuntimeError):
    """A kernel of this library reported a failure (bad argument, CUDA error, bounded wait ran out)."""


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        if not os.path.exists(LIB_PATH):
            raise KernelError(
                f"{LIB_PATH} is missing: build it with `python -m pippy_b200.csrc.build` "
                "(CUDA tensors have no eager fallback in this package)"
            )
        handle = ctypes.CDLL(LIB_PATH)
        handle.pb_launch_count.restype = c_ll
        handle.pb_last_cuda_error.restype = ctypes.c_char_p
        _LIB = handle
    return _LIB


def available() -> bool:
    return os.path.exists(LIB_PATH)


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def err_word(device: torch.device | None = None) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait runs out."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    w = _ERR_WORDS.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _ERR_WORDS[idx] = w
        if lib().pb_bounds_check_enabled():
            # debug build: kernels without an error-word argument of their own report through this one
            lib().pb_set_debug_err_ptr(c_void_p(w.data_ptr()))
    return w


def bounds_check_enabled() -> bool:
    """True when the library was built with ``PIPPY_BOUNDS_CHECK=1`` (index validation in the kernels)."""
    return bool(available() and lib().pb_bounds_check_enabled())


def check_device_errors() -> None:
    """Synchronises and raises :class:`KernelError` if any kernel flagged an error since the last check."""
    for idx, w in _ERR_WORDS.items():
        code = int(w.item())
        if code != 0:
            w.zero_()
            raise KernelError(f"device {idx}: kernel error code {code} (1 = bounded wait ran out, 3 = peer wait ran out, "
                              "4 = MoE receive buffer overflow, 5 = index out of range in a bounds-checking build)")


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().pb_last_cuda_error().decode() if rc > 0 else "invalid argument"
        raise KernelError(f"{what} failed with code {rc}: {msg}")


def launch_count() -> int:
    return int(lib().pb_launch_count()) if available() else 0


def reset_launch_count() -> None:
    if available():
        lib().pb_launch_count_reset()
