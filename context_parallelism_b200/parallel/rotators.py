"""K/V block rotators over ``torch.distributed`` — the NCCL-only baseline transport.

Three strategies with one interface, as in the reference (context_parallel/RingRotator.h:90-447):
``p2p`` (paired send/recv to next/from previous), ``alltoall`` (a sparse all-to-all with a single
non-zero split) and ``allgather`` (one all-gather up front, then block ``(rank - step) mod N`` is just
an index).  ``exchange(buf)`` starts moving ``buf`` to the next rank and returns a handle whose
``wait()`` yields the block received from the previous rank; compute on the current block overlaps
the transfer.  Works on NCCL (GPU) and gloo (CPU) groups.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


class _Handle:
    def __init__(self, works, recv):
        self.works, self.recv = works, recv

    def wait(self) -> torch.Tensor:
        for w in self.works:
            w.wait()
        return self.recv


class _NativeHandle:
    """Handle of a hop on the native process group: the consumer's stream waits on the device for the work's event
    (``Work::streamWait`` of the reference, process_group/CpuSync_fixed.hpp:174-187); the send buffer is kept alive
    until then."""

    def __init__(self, work, recv, keep):
        self.work, self.recv, self.keep = work, recv, keep

    def wait(self) -> torch.Tensor:
        self.work.stream_wait(torch.cuda.current_stream(self.recv.device))
        self.recv.record_stream(torch.cuda.current_stream(self.recv.device))
        self.work.close()
        self.keep = None
        return self.recv


# torch group (by id) -> native process group with a dedicated ring communicator (registered by CPContext on CUDA)
NATIVE_GROUPS = {}


class P2PRotator:
    name = "p2p"

    def __init__(self, group, reverse: bool = False):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        ranks = dist.get_process_group_ranks(group)
        self.reverse = reverse
        step = -1 if reverse else 1
        self.next = ranks[(self.rank + step) % self.size]
        self.prev = ranks[(self.rank - step) % self.size]

    def exchange(self, buf: torch.Tensor) -> _Handle:
        recv = torch.empty_like(buf)
        native = NATIVE_GROUPS.get(id(self.group)) if buf.is_cuda else None
        if native is not None:
            step = -1 if self.reverse else 1
            buf = buf.contiguous()
            w = native.sendrecv(buf, recv, (self.rank + step) % self.size, (self.rank - step) % self.size)
            return _NativeHandle(w, recv, buf)
        ops = [dist.P2POp(dist.isend, buf, self.next, self.group), dist.P2POp(dist.irecv, recv, self.prev, self.group)]
        return _Handle(dist.batch_isend_irecv(ops), recv)


class AllToAllRotator:
    name = "alltoall"

    def __init__(self, group, reverse: bool = False):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        step = -1 if reverse else 1
        self.next = (self.rank + step) % self.size
        self.prev = (self.rank - step) % self.size

    def exchange(self, buf: torch.Tensor) -> _Handle:
        flat = buf.reshape(-1)
        recv = torch.empty_like(flat)
        n = flat.numel()
        in_split = [n if r == self.next else 0 for r in range(self.size)]
        out_split = [n if r == self.prev else 0 for r in range(self.size)]
        w = dist.all_to_all_single(recv, flat, out_split, in_split, group=self.group, async_op=True)
        return _Handle([w], recv.view(buf.shape))


class AllGatherRotator:
    """Gathers every rank's block once; ``block(step)`` is then an index (fp32/bf16 alike)."""
    name = "allgather"

    def __init__(self, group, reverse: bool = False):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.gathered: Optional[List[torch.Tensor]] = None
        self.step = 0
        self.reverse = reverse

    def exchange(self, buf: torch.Tensor) -> _Handle:
        if self.gathered is None:
            full = torch.empty((self.size,) + tuple(buf.shape), dtype=buf.dtype, device=buf.device)
            dist.all_gather_into_tensor(full.view(-1), buf.reshape(-1).contiguous(), group=self.group)
            self.gathered = full
            self.step = 0
        self.step += 1
        src = (self.rank + self.step) % self.size if self.reverse else (self.rank - self.step) % self.size
        return _Handle([], self.gathered[src])

    def reset(self) -> None:
        self.gathered, self.step = None, 0


def make_rotator(kind: str, group, reverse: bool = False):
    if kind == "p2p":
        return P2PRotator(group, reverse)
    if kind == "alltoall":
        return AllToAllRotator(group, reverse)
    if kind == "allgather":
        return AllGatherRotator(group, reverse)
    raise ValueError(f"unknown rotator {kind!r}")
