"""Symmetric (peer-mapped) device memory for the fused communication kernels.

Every rank of a node allocates the same number of bytes with ``cudaMalloc`` (through the package's library, so the
allocation is IPC-exportable whatever the PyTorch allocator is configured to do), the 64-byte IPC handles travel
over the process group's side channel, and each rank maps all peers' allocations.  Kernels then receive an array of
``world`` base pointers and load/store the peers' memory directly over NVLink.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib


class _CudaArray:
    """Minimal ``__cuda_array_interface__`` holder so torch can view raw device memory without copying."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }
        self._owner = owner


class SymmetricBuffer:
    """``nbytes`` of zero-initialised device memory on every rank of ``group``, mapped everywhere."""

    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        lib = _lib.lib()
        with torch.cuda.device(self.device):
            base = ctypes.c_void_p()
            _lib.check(lib.pb_peer_alloc(ctypes.c_ulonglong(self.nbytes), ctypes.byref(base)), "pb_peer_alloc")
            self.local_ptr = int(base.value)
            hbytes = int(lib.pb_ipc_handle_bytes())
            handle = ctypes.create_string_buffer(hbytes)
            _lib.check(lib.pb_ipc_get_handle(ctypes.c_void_p(self.local_ptr), handle), "pb_ipc_get_handle")
            handles: List[Optional[bytes]] = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, handle.raw, group=group)
            else:
                handles = [handle.raw]
            self.ptrs: List[int] = []
            self._opened: List[int] = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(self.local_ptr)
                    continue
                out = ctypes.c_void_p()
                _lib.check(lib.pb_ipc_open(ctypes.c_char_p(h), ctypes.byref(out)), "pb_ipc_open")
                self.ptrs.append(int(out.value))
                self._opened.append(int(out.value))
        self._view = torch.as_tensor(_CudaArray(self.local_ptr, self.nbytes, self), device=self.device)
        if self.world > 1:
            dist.barrier(group=group)

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        """A tensor view of this rank's own buffer."""
        item = torch.empty((), dtype=dtype).element_size()
        avail = (self.nbytes - offset_bytes) // item
        n = avail if numel is None else numel
        if n > avail:
            raise ValueError(f"view of {n} x {dtype} does not fit the {self.nbytes}-byte buffer")
        return self._view[offset_bytes : offset_bytes + n * item].view(dtype)

    def pointer_array(self, offset_bytes: int = 0):
        """ctypes array of ``world`` pointers (every rank's base + offset), in rank order."""
        arr = (ctypes.c_void_p * self.world)()
        for i, p in enumerate(self.ptrs):
            arr[i] = ctypes.c_void_p(p + offset_bytes)
        return arr

    def close(self) -> None:
        lib = _lib.lib()
        for p in self._opened:
            lib.pb_ipc_close(ctypes.c_void_p(p))
        self._opened = []
        if self.local_ptr:
            self._view = None
            lib.pb_peer_free(ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0
