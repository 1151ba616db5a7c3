"""Symmetric peer-memory heap (one node, NVLink/NVSwitch) and the kernels' synchronisation flags.

Every rank of a group allocates an arena of the same size (``csrc/runtime/symm.cpp``), the CUDA IPC
handles are exchanged once through the process group, and each rank maps every peer's arena.  A
sub-allocation has the same offset on every rank, so a kernel reaches a peer's copy of a buffer at
``peer_base[rank] + offset`` with plain loads/stores.  Flags (int32) live in the same arena;
"epochs" grow monotonically so flags are never reset.

Only same-node groups are supported (CUDA IPC); the fused kernels are used only then.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native as nv


class _RawCuda:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    """uint8 tensor aliasing raw device memory (not owned by the PyTorch allocator)."""
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=device)


class SymmetricHeap:
    def __init__(self, group, nbytes: int, device: torch.device):
        self.group = group
        self.device = device
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = (nbytes + 4095) // 4096 * 4096
        base = ctypes.c_void_p()
        nv.check(nv.lib().cpb_symm_alloc(ctypes.c_size_t(self.nbytes), ctypes.byref(base)), "symm_alloc")
        self.base = base.value
        handle = (ctypes.c_ubyte * 64)()
        nv.check(nv.lib().cpb_symm_export(ctypes.c_void_p(self.base), handle), "symm_export")
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.peer_bases: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peer_bases.append(self.base)
                continue
            p = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            nv.check(nv.lib().cpb_symm_import(buf, ctypes.byref(p)), "symm_import")
            self.peer_bases.append(p.value)
            self._opened.append(p.value)
        self.peer_table = torch.tensor(self.peer_bases, dtype=torch.int64, device=device)
        self.arena = tensor_from_ptr(self.base, self.nbytes, device)
        self._off = 0
        self._named: Dict[str, Tuple[int, int]] = {}
        dist.barrier(group=group)

    def alloc(self, name: str, nbytes: int, align: int = 1024) -> int:
        """Reserve ``nbytes`` (same call order and sizes on every rank) and return its arena offset."""
        if name in self._named:
            off, size = self._named[name]
            if size < nbytes:
                raise RuntimeError(f"symmetric buffer {name!r} was reserved with {size} bytes, {nbytes} requested")
            return off
        off = (self._off + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise RuntimeError(f"symmetric heap exhausted: {off + nbytes} > {self.nbytes} bytes (buffer {name!r})")
        self._off = off + nbytes
        self._named[name] = (off, nbytes)
        return off

    def view(self, off: int, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self.arena[off:off + nb].view(dtype).view(*shape)

    def tensor(self, name: str, shape, dtype: torch.dtype) -> Tuple[torch.Tensor, int]:
        n = 1
        for s in shape:
            n *= s
        off = self.alloc(name, n * torch.empty((), dtype=dtype).element_size())
        return self.view(off, shape, dtype), off

    def raw_tensor(self, name: str, shape, dtype: torch.dtype) -> Tuple[torch.Tensor, int]:
        """Like :meth:`tensor`, but the result is a tensor object of its own over the arena memory (own storage
        object, own autograd version counter): in-place writes elsewhere in the arena do not invalidate it for
        autograd.  Used for buffers that parameters are views of."""
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        off = self.alloc(name, nb)
        return tensor_from_ptr(self.base + off, nb, self.device).view(dtype).view(*shape), off

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        if dist.is_initialized():
            try:
                dist.barrier(group=self.group)
            except Exception:
                pass
        for p in self._opened:
            nv.lib().cpb_symm_close(ctypes.c_void_p(p))
        self._opened = []
        if self.base:
            self.arena = None
            nv.lib().cpb_symm_free(ctypes.c_void_p(self.base))
            self.base = 0
