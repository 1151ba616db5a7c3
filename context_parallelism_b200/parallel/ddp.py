"""Bucketed parameter-gradient all-reduce overlapped with backward.

Gradients live in one flat fp32 buffer (``ops.optim.FlatParams``); it is cut into buckets of about
``CP_GRAD_BUCKET_MB`` (25 MB, the reference's DDP bucket size, Scripts/Blutrain/bluscriptCP.cpp:1003-1012).
Our backward kernels call ``param._grad_ready`` when a parameter's gradient is final; when every
parameter of a bucket has reported, the bucket's all-reduce starts on a side stream while backward
continues.  ``finish()`` joins the side stream before the optimiser runs.  During gradient
accumulation ``no_sync`` suppresses communication until the last micro-batch (the reference's
``ddp.no_sync()`` / ``ddp.sync()``, bluscriptCP.cpp:1698-1716).

Reduction is an AVERAGE over every rank of the group (all dp·cp ranks: each rank's loss is a mean over
its own tokens, Scripts/Blutrain/gpt2_cp_test.cpp:1574-1601; context_parallel/RopeGammaAccum.h:16-21).

Transports: ``nccl`` (``dist.all_reduce``; baseline, also used on gloo/CPU) or ``fused`` (the peer-memory
kernels of ``parallel.fused``).  With the sharded optimiser (the default of the fused transport) a bucket is only
reduce-scattered: every rank reduces the sub-slice it owns straight from the peers' fp32 gradient buffers, and its
AdamW consumes that shard; with ``CP_SHARD_OPTIM=0`` the two-shot all-reduce (cast/scale + reduce + gather) runs.
"""
from __future__ import annotations

import contextlib
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class GradReducer:
    def __init__(self, flat, group, world: int, bucket_mb: int = 25, fused=None, overlap: bool = True):
        self.flat, self.group, self.world = flat, group, world
        self.fused = fused
        self.enabled = world > 1
        self.sync_enabled = True
        self.overlap = overlap and flat.device.type == "cuda"
        # buckets are contiguous ranges of the flat buffer, cut at parameter boundaries (planned by FlatParams so the
        # sharded optimiser and the reducer agree on them)
        self.buckets: List[List[int]] = [[s, e] for s, e in flat.buckets]
        self.param_bucket: Dict[int, int] = {}
        starts = [b[0] for b in self.buckets]
        import bisect
        for name, p, off, n in flat.entries:
            self.param_bucket[id(p)] = bisect.bisect_right(starts, off) - 1
        self.expected: Optional[Dict[int, int]] = None      # hook invocations per parameter in one backward
        self._calls: Dict[int, int] = {}
        self._seen: List[int] = [0] * len(self.buckets)
        self._launched: List[bool] = [False] * len(self.buckets)
        self.stream = torch.cuda.Stream(device=flat.device) if self.overlap else None
        self._pending = []
        if self.enabled:
            for _, p, _, _ in flat.entries:
                p._grad_ready = self._on_ready

    @contextlib.contextmanager
    def no_sync(self):
        prev, self.sync_enabled = self.sync_enabled, False
        try:
            yield
        finally:
            self.sync_enabled = prev

    # ------------------------------------------------------------------ backward-time hooks
    def begin_backward(self) -> None:
        self._calls = {}
        self._seen = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)

    def _on_ready(self, p) -> None:
        if not (self.enabled and self.sync_enabled):
            return
        pid = id(p)
        self._calls[pid] = self._calls.get(pid, 0) + 1
        if self.expected is None or not self.overlap:
            return
        if self._calls[pid] == self.expected.get(pid, 1):
            b = self.param_bucket[pid]
            self._seen[b] += 1
            if self._seen[b] == self._bucket_nparams(b) and not self._launched[b]:
                self._launch(b)

    def _bucket_nparams(self, b: int) -> int:
        if not hasattr(self, "_nparams"):
            self._nparams = [0] * len(self.buckets)
            for pid, bi in self.param_bucket.items():
                self._nparams[bi] += 1
        return self._nparams[b]

    def _launch(self, b: int) -> None:
        self._launched[b] = True
        s, e = self.buckets[b]
        buf = self.flat.grad[s:e]
        if self.stream is not None:
            self.stream.wait_stream(torch.cuda.current_stream(self.flat.device))
            with torch.cuda.stream(self.stream):
                self._allreduce(buf, s, b)
        else:
            self._allreduce(buf, s, b)

    def _allreduce(self, buf: torch.Tensor, offset: int, b: int) -> None:
        if self.fused is not None and buf.is_cuda and self.flat.sharded:
            self.fused.reduce_scatter_bucket(self.flat, b)       # the owner's AdamW consumes the reduced shard
        elif self.fused is not None and buf.is_cuda:
            self.fused.allreduce_avg_(buf, offset)
        else:
            dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.group)
            buf.mul_(1.0 / self.world)

    # ------------------------------------------------------------------ end of backward
    def finish(self) -> None:
        """Reduce whatever has not been launched yet and make the compute stream wait for all of it."""
        if not (self.enabled and self.sync_enabled):
            return
        if self.expected is None:
            self.expected = dict(self._calls)       # learnt from the first full backward
        for b in range(len(self.buckets)):
            if not self._launched[b]:
                self._launch(b)
        if self.fused is not None:
            if self.stream is not None:
                with torch.cuda.stream(self.stream):
                    self.fused.allreduce_finish()
            else:
                self.fused.allreduce_finish()
        if self.stream is not None:
            torch.cuda.current_stream(self.flat.device).wait_stream(self.stream)

    def broadcast_params(self, src: int = 0) -> None:
        """Initial parameter sync from rank ``src`` of the group (DDP ``init_sync``, bluscriptCP.cpp:1011)."""
        if not self.enabled:
            return
        if self.flat.sharded:
            raise RuntimeError("broadcast_params: with a sharded optimiser broadcast the model parameters before packing them")
        ranks = dist.get_process_group_ranks(self.group) if self.group is not None else None
        gsrc = ranks[src] if ranks is not None else src
        dist.broadcast(self.flat.master, gsrc, group=self.group)
        self.flat.sync_compute_copy()
