"""Python face of the native NCCL process group (``csrc/runtime/process_group.cpp``).

A group owns a collective communicator and a dedicated ring communicator with its own stream; every call returns a
``Work`` (``parallel.work``) that the caller waits on the device (``stream_wait``) or on the host with the
``CP_WATCHDOG_S`` deadline.  The NCCL unique ids are made on the group's first rank and handed round through
``torch.distributed`` (bootstrap only; the reference used ``MPI_Bcast``, process_group/processGroupNCCL.cpp:62,118).
Used by the NCCL baseline transports (``parallel.rotators``); the product paths use the peer-memory kernels.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as nv
from .work import Work

_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.int32: 3, torch.int64: 4, torch.uint8: 5, torch.float64: 6}
_OPS = {"sum": 0, "avg": 1, "max": 2, "min": 3, "prod": 4}


def _work(h: ctypes.c_void_p) -> Work:
    w = Work.__new__(Work)
    w._h = h
    return w


class NativeProcessGroup:
    def __init__(self, handle: ctypes.c_void_p, world: int, rank: int, device: torch.device):
        self._h, self.world, self.rank, self.device = handle, world, rank, device

    @staticmethod
    def create(torch_group=None, timeout_s: float = 600.0, with_ring: bool = True,
               device: Optional[torch.device] = None) -> "NativeProcessGroup":
        """Collective over ``torch_group`` (default: the world): every member calls this."""
        lib = nv.lib()
        device = device or torch.device("cuda", torch.cuda.current_device())
        world, rank = dist.get_world_size(torch_group), dist.get_rank(torch_group)
        ids = [None, None]
        if rank == 0:
            for i in range(2 if with_ring else 1):
                buf = (ctypes.c_ubyte * 128)()
                nv.check(lib.cpb_pg_unique_id(buf), "pg_unique_id")
                ids[i] = bytes(buf)
        src = dist.get_process_group_ranks(torch_group)[0] if torch_group is not None else 0
        dist.broadcast_object_list(ids, src=src, group=torch_group)
        h = ctypes.c_void_p()
        a = (ctypes.c_ubyte * 128).from_buffer_copy(ids[0])
        b = (ctypes.c_ubyte * 128).from_buffer_copy(ids[1]) if ids[1] is not None else None
        with torch.cuda.device(device):
            nv.check(lib.cpb_pg_create(a, b, ctypes.c_int(world), ctypes.c_int(rank), ctypes.c_double(timeout_s), ctypes.byref(h)), "pg_create")
        return NativeProcessGroup(h, world, rank, device)

    def split(self, color: int, key: int, new_world: int, new_rank: int) -> "NativeProcessGroup":
        """``ncclCommSplit``: ranks with the same colour form a sub-group ordered by key (every rank of this group calls)."""
        h = ctypes.c_void_p()
        nv.check(nv.lib().cpb_pg_split(self._h, ctypes.c_int(color), ctypes.c_int(key), ctypes.c_int(new_world), ctypes.c_int(new_rank),
                                       ctypes.byref(h)), "pg_split")
        return NativeProcessGroup(h, new_world, new_rank, self.device)

    # ------------------------------------------------------------------ collectives (all asynchronous)
    def _s(self) -> ctypes.c_void_p:
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def all_reduce(self, t: torch.Tensor, op: str = "sum") -> Work:
        h = ctypes.c_void_p()
        nv.check(nv.lib().cpb_pg_all_reduce(self._h, nv.ptr(t), nv.l(t.numel()), nv.i(_DTYPES[t.dtype]), nv.i(_OPS[op]), self._s(), ctypes.byref(h)), "pg_all_reduce")
        return _work(h)

    def broadcast(self, t: torch.Tensor, root: int = 0) -> Work:
        h = ctypes.c_void_p()
        nv.check(nv.lib().cpb_pg_broadcast(self._h, nv.ptr(t), nv.l(t.numel()), nv.i(_DTYPES[t.dtype]), nv.i(root), self._s(), ctypes.byref(h)), "pg_broadcast")
        return _work(h)

    def all_gather(self, send: torch.Tensor, recv: torch.Tensor) -> Work:
        assert recv.numel() == send.numel() * self.world and send.is_contiguous() and recv.is_contiguous()
        h = ctypes.c_void_p()
        nv.check(nv.lib().cpb_pg_all_gather(self._h, nv.ptr(send), nv.ptr(recv), nv.l(send.numel()), nv.i(_DTYPES[send.dtype]), self._s(), ctypes.byref(h)), "pg_all_gather")
        return _work(h)

    def reduce_scatter(self, send: torch.Tensor, recv: torch.Tensor, op: str = "sum") -> Work:
        assert send.numel() == recv.numel() * self.world and send.is_contiguous() and recv.is_contiguous()
        h = ctypes.c_void_p()
        nv.check(nv.lib().cpb_pg_reduce_scatter(self._h, nv.ptr(send), nv.ptr(recv), nv.l(recv.numel()), nv.i(_DTYPES[send.dtype]), nv.i(_OPS[op]),
                                                self._s(), ctypes.byref(h)), "pg_reduce_scatter")
        return _work(h)

    def all_to_all(self, send: torch.Tensor, recv: torch.Tensor) -> Work:
        assert send.numel() == recv.numel() and send.numel() % self.world == 0 and send.is_contiguous() and recv.is_contiguous()
        h = ctypes.c_void_p()
        nv.check(nv.lib().cpb_pg_all_to_all(self._h, nv.ptr(send), nv.ptr(recv), nv.l(send.numel() // self.world), nv.i(_DTYPES[send.dtype]),
                                            self._s(), ctypes.byref(h)), "pg_all_to_all")
        return _work(h)

    def sendrecv(self, send: torch.Tensor, recv: torch.Tensor, dst: int, src: int) -> Work:
        """One ring hop on the dedicated ring communicator and stream."""
        assert send.numel() == recv.numel() and send.is_contiguous() and recv.is_contiguous()
        h = ctypes.c_void_p()
        nv.check(nv.lib().cpb_pg_sendrecv(self._h, nv.ptr(send), nv.ptr(recv), nv.l(send.numel()), nv.i(_DTYPES[send.dtype]), nv.i(dst), nv.i(src),
                                          self._s(), ctypes.byref(h)), "pg_sendrecv")
        return _work(h)

    # ------------------------------------------------------------------ failure handling / teardown
    def async_error(self) -> int:
        return int(nv.lib().cpb_pg_async_error(self._h))

    def abort(self) -> None:
        nv.lib().cpb_pg_abort(self._h)

    def close(self) -> None:
        if self._h is not None:
            nv.lib().cpb_pg_destroy(self._h)
            self._h = None
