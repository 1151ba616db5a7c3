"""Flat parameter storage, fused gradient-norm clipping and AdamW, replicated or sharded over the ranks.

``FlatParams`` packs every parameter of a model into a few flat buffers.  Parameters become views of the
compute copies (bf16 for matrices, fp32 for vectors); ``p.main_grad`` is the fp32 gradient view our backward
kernels accumulate into directly.  Two layouts:

* **replicated** (one rank, the CPU oracle, the NCCL baseline): fp32 master weights, gradients and Adam moments
  for every parameter on every rank — what the reference does (``DataParallel`` + ``nn::AdamW`` on every rank,
  Scripts/Blutrain/bluscriptCP.cpp:1003-1017,1742-1744).
* **sharded** (the fused peer-memory transport): the gradient all-reduce becomes reduce-scatter → AdamW on the
  owned slice → all-gather of the updated parameters.  The flat index space is cut into buckets (the gradient
  buckets of ``parallel.ddp``) and rank r owns the r-th sub-slice of every bucket, so every bucket's reduction
  uses every NVLink at once.  fp32 master / m / v exist only for the owned slices (12 bytes per parameter divided
  by the number of ranks); the full-length buffers that remain are the fp32 gradient (4 B) and the bf16 compute
  copy (2 B), both inside the symmetric arena so peers can read them.  The replicated tail of the step (every rank
  running AdamW and the norm over all parameters) disappears, and because exactly one rank computes each
  parameter's update from fp32 sums taken in a fixed order, the replicas cannot drift apart.

One ``sumsq`` launch gives the gradient norm on the device, and one ``adamw`` launch applies clip + decoupled
weight decay + Adam and refreshes the compute copy, with no host synchronisation (the reference does
``clip_grad_norm_``, a manual decay loop over parameters and ``AdamW.step``, bluscriptCP.cpp:1736-1744).  A
non-finite norm skips the step and sets a flag instead of poisoning the weights (the reference aborts on a NaN
loss, bluscriptCP.cpp:1730-1733).

Semantics follow ``torch.optim.AdamW`` (bias correction, eps outside the square root, decay on parameters with
``dim >= 2`` only).
"""
from __future__ import annotations

import bisect
import math
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .. import _native as nv
from . import reference as ref


def _pad64(n: int) -> int:
    return (n + 63) // 64 * 64


def plan_buckets(entries, total: int, bucket_elems: int) -> List[Tuple[int, int]]:
    """Contiguous ``(start, end)`` ranges of the flat buffer of at least ``bucket_elems`` elements, cut at
    parameter boundaries (25 MB by default, the reference's DDP bucket size, bluscriptCP.cpp:1003-1012)."""
    out, start = [], 0
    for _, _, off, n in entries:
        end = off + _pad64(n)
        if end - start >= bucket_elems:
            out.append((start, end))
            start = end
    if start < total:
        out.append((start, total))
    return out


class ShardPlan:
    """Ownership of the flat index space: inside bucket ``(start, end)`` rank r owns
    ``[start + r*per, min(end, start + (r+1)*per))`` with ``per = ceil((end-start)/world)`` rounded up to 8
    elements; the owned runs of all buckets are concatenated (each padded to ``per``) into the shard buffers."""

    def __init__(self, buckets: List[Tuple[int, int]], world: int, rank: int):
        self.world, self.rank = world, rank
        self.buckets = []                    # (start, n, per, shard_off)
        off = 0
        for s, e in buckets:
            n = e - s
            per = ((n + world - 1) // world + 7) // 8 * 8
            self.buckets.append((s, n, per, off))
            off += per
        self.shard_total = off

    def owned(self, rank: Optional[int] = None) -> List[Tuple[int, int, int]]:
        """``(flat_begin, flat_end, shard_begin)`` runs of ``rank`` (default: this rank), sorted by flat index."""
        r = self.rank if rank is None else rank
        out = []
        for s, n, per, off in self.buckets:
            a, c = s + r * per, min(s + n, s + (r + 1) * per)
            if c > a:
                out.append((a, c, off))
        return out


class FlatParams:
    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], bf16_matrices: bool,
                 bucket_mb: int = 25, shard=None, bucket_elems: Optional[int] = None):
        """``shard``: the peer-memory transport (``parallel.fused.FusedComm``) when the optimiser state is to be
        sharded over its world group; ``None`` keeps everything replicated.  ``bucket_elems`` overrides the bucket size
        given in MB (tests use tiny buckets)."""
        seen, decay, nodecay = set(), [], []
        for name, p in named_params:
            if id(p) in seen or not p.requires_grad:
                continue
            seen.add(id(p))
            (decay if p.dim() >= 2 else nodecay).append((name, p))
        self.entries: List[Tuple[str, torch.nn.Parameter, int, int]] = []
        off = 0
        for name, p in decay + nodecay:
            n = p.numel()
            self.entries.append((name, p, off, n))
            off += _pad64(n)                    # keep every view 256-byte aligned
        self.n_decay = sum(_pad64(p.numel()) for _, p in decay)
        self.total = off
        dev = (decay + nodecay)[0][1].device
        self.device = dev
        self.bf16 = bool(bf16_matrices and dev.type == "cuda")
        self.buckets = plan_buckets(self.entries, self.total, bucket_elems or max(1, bucket_mb) * (1 << 20) // 4)
        self.shard = shard if (shard is not None and dev.type == "cuda" and self.bf16) else None
        self.plan: Optional[ShardPlan] = None
        self._by_name = {name: (p, o, n) for name, p, o, n in self.entries}
        if self.shard is None:
            self._init_replicated()
        else:
            self._init_sharded()
        self._scratch = torch.zeros(1024 + 8, dtype=torch.float32, device=dev)
        self._ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.skip_flag = torch.zeros(1, dtype=torch.int32, device=dev)

    # ------------------------------------------------------------------ construction
    def _init_replicated(self) -> None:
        dev = self.device
        self.master = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.grad = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.m = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.p16 = torch.zeros(self.n_decay, dtype=torch.bfloat16, device=dev) if self.bf16 else None
        self.p32 = None
        for name, p, o, n in self.entries:
            self.master[o:o + n].copy_(p.detach().reshape(-1).float())
            if self.bf16 and p.dim() >= 2:
                self.p16[o:o + n].copy_(p.detach().reshape(-1))
                p.data = self.p16[o:o + n].view(p.shape)
            else:
                p.data = self.master[o:o + n].view(p.shape)
            self._bind_grad(p, o, n)

    def _init_sharded(self) -> None:
        dev, fc = self.device, self.shard
        self.plan = plan = ShardPlan(self.buckets, fc.shard_world, fc.shard_rank)
        self.grad, self.grad_off = fc.heap.raw_tensor("flat.grad", (self.total,), torch.float32)
        self.p16, self.p16_off = fc.heap.raw_tensor("flat.p16", (max(self.n_decay, 8),), torch.bfloat16)
        self.p32, self.p32_off = fc.heap.raw_tensor("flat.p32", (max(self.total - self.n_decay, 8),), torch.float32)
        self.slots, self.slots_off = fc.heap.raw_tensor("flat.norm_slots", (64,), torch.float32)
        self.grad.zero_(); self.p16.zero_(); self.p32.zero_(); self.slots.zero_()
        st = plan.shard_total
        self.master = torch.zeros(st, dtype=torch.float32, device=dev)
        self.m = torch.zeros(st, dtype=torch.float32, device=dev)
        self.v = torch.zeros(st, dtype=torch.float32, device=dev)
        self.gshard = torch.zeros(st, dtype=torch.float32, device=dev)
        self._owned = plan.owned()
        self._owned_starts = [a for a, _, _ in self._owned]
        for name, p, o, n in self.entries:
            src = p.detach().reshape(-1).float()
            self._scatter(self.master, o, src)
            if p.dim() >= 2:
                self.p16[o:o + n].copy_(src)
                p.data = self.p16[o:o + n].view(p.shape)
            else:
                q = o - self.n_decay
                self.p32[q:q + n].copy_(src)
                p.data = self.p32[q:q + n].view(p.shape)
            self._bind_grad(p, o, n)
        # device tables of the optimiser and all-gather launches
        adam, g16, g32 = [], [], []
        for a, c, sb in self._owned:
            for lo, hi, dec in ((a, min(c, self.n_decay), 1), (max(a, self.n_decay), c, 0)):
                if hi > lo:
                    adam.append([sb + (lo - a), lo, hi - lo, dec])
        for s, n, per, _ in plan.buckets:
            lo, hi = s, min(s + n, self.n_decay)
            if hi > lo:
                g16.append([lo, hi - lo, s, per])
            lo, hi = max(s, self.n_decay), s + n
            if hi > lo:
                g32.append([lo, hi - lo, s, per])
        t = lambda rows: torch.tensor(rows, dtype=torch.int64, device=dev) if rows else None     # noqa: E731
        self._adam_segs, self._g16_segs, self._g32_segs = t(adam), t(g16), t(g32)

    def _bind_grad(self, p, o: int, n: int) -> None:
        gview = self.grad[o:o + n].view(p.shape)
        if self.device.type == "cuda":
            p.main_grad = gview
        else:
            p.grad = gview

    # ------------------------------------------------------------------ shard <-> flat index helpers
    def _scatter(self, shard_buf: torch.Tensor, flat_lo: int, values: torch.Tensor) -> None:
        """Copy ``values`` (flat indices ``flat_lo ...``) into the parts of ``shard_buf`` this rank owns."""
        flat_hi = flat_lo + values.numel()
        i = max(0, bisect.bisect_right(self._owned_starts, flat_lo) - 1)
        while i < len(self._owned) and self._owned[i][0] < flat_hi:
            a, c, sb = self._owned[i]
            lo, hi = max(a, flat_lo), min(c, flat_hi)
            if hi > lo:
                shard_buf[sb + lo - a: sb + hi - a].copy_(values[lo - flat_lo: hi - flat_lo])
            i += 1

    def _full_from_shards(self, shard_buf: torch.Tensor) -> torch.Tensor:
        """Flat fp32 tensor assembled from every rank's shard (a collective over the transport's world group)."""
        import torch.distributed as dist
        plan = self.plan
        gathered = torch.empty(plan.world * plan.shard_total, dtype=shard_buf.dtype, device=self.device)
        dist.all_gather_into_tensor(gathered, shard_buf.contiguous(), group=self.shard.world_group)
        full = torch.zeros(self.total, dtype=shard_buf.dtype, device=self.device)
        for s, n, per, off in plan.buckets:
            for r in range(plan.world):
                a, c = s + r * per, min(s + n, s + (r + 1) * per)
                if c > a:
                    full[a:c].copy_(gathered[r * plan.shard_total + off: r * plan.shard_total + off + (c - a)])
        return full

    # ------------------------------------------------------------------ helpers
    @property
    def sharded(self) -> bool:
        return self.plan is not None

    def zero_grad(self) -> None:
        self.grad.zero_()

    def full_master(self) -> torch.Tensor:
        """All fp32 master weights as one flat tensor (collective when sharded)."""
        return self._full_from_shards(self.master) if self.sharded else self.master

    def full_moments(self) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.sharded:
            return self._full_from_shards(self.m), self._full_from_shards(self.v)
        return self.m, self.v

    def full_reduced_grad(self) -> torch.Tensor:
        """The averaged gradient after the reduction of a step (collective when sharded)."""
        return self._full_from_shards(self.gshard) if self.sharded else self.grad

    def named_master(self) -> Dict[str, torch.Tensor]:
        full = self.full_master()
        return {name: full[o:o + n].view(p.shape) for name, p, o, n in self.entries}

    def sync_compute_copy(self) -> None:
        """Refresh the compute copies from the fp32 masters (replicated layout; the sharded layout refreshes them in
        ``load_master_rows``)."""
        if self.bf16 and not self.sharded:
            self.p16.copy_(self.master[: self.n_decay])

    def load_master_rows(self, name: str, row0: int, value: torch.Tensor) -> None:
        """Overwrite rows ``row0 ...`` of parameter ``name`` (all of it for vectors) with ``value`` (every rank
        calls this with the same data) and refresh the compute copy."""
        p, o, n = self._by_name[name]
        cols = p.shape[1] if p.dim() >= 2 else 1
        lo = o + row0 * cols
        src = value.reshape(-1).to(device=self.device, dtype=torch.float32)
        if lo + src.numel() > o + n:
            raise ValueError(f"{name}: {src.numel()} values at row {row0} exceed the parameter")
        if self.sharded:
            self._scatter(self.master, lo, src)
            if p.dim() >= 2:
                self.p16[lo:lo + src.numel()].copy_(src)
            else:
                self.p32[lo - self.n_decay: lo - self.n_decay + src.numel()].copy_(src)
        else:
            self.master[lo:lo + src.numel()].copy_(src)
            if self.bf16 and p.dim() >= 2:
                self.p16[lo:lo + src.numel()].copy_(src)

    def load_master(self, name: str, value: torch.Tensor) -> None:
        self.load_master_rows(name, 0, value)

    def load_moments(self, name: str, m: torch.Tensor, v: torch.Tensor) -> None:
        p, o, n = self._by_name[name]
        mm = m.reshape(-1).to(device=self.device, dtype=torch.float32)
        vv = v.reshape(-1).to(device=self.device, dtype=torch.float32)
        if self.sharded:
            self._scatter(self.m, o, mm)
            self._scatter(self.v, o, vv)
        else:
            self.m[o:o + n].copy_(mm)
            self.v[o:o + n].copy_(vv)

    def local_sumsq_(self) -> None:
        """Sum of squares of what this rank holds of the (reduced) gradient into ``self.sumsq`` (device, no sync)."""
        if self.sharded:
            nv.call("sumsq", nv.ptr(self.gshard), nv.l(self.plan.shard_total), nv.ptr(self._scratch), nv.ptr(self._ticket),
                    nv.ptr(self.sumsq), nv.stream_ptr(self.device))
        elif self.device.type == "cuda":
            nv.call("sumsq", nv.ptr(self.grad), nv.l(self.total), nv.ptr(self._scratch), nv.ptr(self._ticket),
                    nv.ptr(self.sumsq), nv.stream_ptr(self.device))
        else:
            self.sumsq[0] = (self.grad.double() ** 2).sum().float()

    def grad_norm(self, prescale: float = 1.0) -> torch.Tensor:
        """Global L2 norm of the (reduced) gradient times ``prescale`` as a device scalar (no host sync)."""
        self.local_sumsq_()
        if self.sharded:
            self.shard.sum_over_ranks_(self.sumsq, self.slots_off, self.slots)
        return self.sumsq.sqrt() * prescale


class AdamW:
    """Fused AdamW over a :class:`FlatParams` (replicated or sharded)."""

    def __init__(self, flat: FlatParams, lr: float, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1):
        self.flat, self.lr, self.betas, self.eps, self.wd = flat, lr, betas, eps, weight_decay
        self.step_count = 0

    def zero_grad(self) -> None:
        self.flat.zero_grad()

    def step(self, lr: Optional[float] = None, clip: float = 0.0, grad_prescale: float = 1.0) -> torch.Tensor:
        """Clip (global norm, on device) and update.  Returns the pre-clip gradient norm (device scalar)."""
        f = self.flat
        lr = self.lr if lr is None else lr
        self.step_count += 1
        norm = f.grad_norm(grad_prescale)
        b1, b2 = self.betas
        if f.sharded:
            self.update_shard_(lr, clip, grad_prescale)
            f.shard.allgather_params(f)
        elif f.device.type == "cuda":
            for lo, hi, wd in ((0, f.n_decay, self.wd), (f.n_decay, f.total, 0.0)):
                if hi <= lo:
                    continue
                p16 = f.p16[lo:hi] if (f.bf16 and hi <= f.n_decay) else None
                nv.call("adamw", nv.ptr(f.master[lo:hi]), nv.ptr(f.grad[lo:hi]), nv.ptr(f.m[lo:hi]), nv.ptr(f.v[lo:hi]),
                        nv.ptr(p16), nv.l(hi - lo), nv.f(lr), nv.f(b1), nv.f(b2), nv.f(self.eps), nv.f(wd),
                        nv.i(self.step_count), nv.f(grad_prescale), nv.f(clip), nv.ptr(f.sumsq), nv.ptr(f.skip_flag),
                        nv.stream_ptr(f.device))
        else:
            nrm = float(norm)
            if not math.isfinite(nrm):
                f.skip_flag[0] = 1
                return norm
            gs = grad_prescale * (min(1.0, clip / (nrm + 1e-6)) if clip > 0 else 1.0)
            g = f.grad * gs
            for lo, hi, wd in ((0, f.n_decay, self.wd), (f.n_decay, f.total, 0.0)):
                if hi > lo:
                    ref.adamw_step(f.master[lo:hi], g[lo:hi], f.m[lo:hi], f.v[lo:hi], self.step_count, lr, b1, b2, self.eps, wd)
        return norm

    def update_shard_(self, lr: float, clip: float, grad_prescale: float = 1.0) -> None:
        """Sharded layout: AdamW on the owned slices, from ``flat.gshard`` and the global squared norm in
        ``flat.sumsq``; writes the refreshed compute copies at their flat positions (one launch)."""
        f = self.flat
        b1, b2 = self.betas
        if f._adam_segs is not None:
            nv.call("adamw_sharded", nv.ptr(f.master), nv.ptr(f.gshard), nv.ptr(f.m), nv.ptr(f.v), nv.ptr(f.p16), nv.ptr(f.p32),
                    nv.l(f.n_decay), nv.ptr(f._adam_segs), nv.i(f._adam_segs.shape[0]), nv.i(16), nv.f(lr), nv.f(b1), nv.f(b2),
                    nv.f(self.eps), nv.f(self.wd), nv.i(self.step_count), nv.f(grad_prescale), nv.f(clip), nv.ptr(f.sumsq),
                    nv.ptr(f.skip_flag), nv.stream_ptr(f.device))

    def state_dict(self) -> Dict[str, torch.Tensor]:
        """Adam moments by parameter name (collective when the state is sharded: call it on every rank)."""
        out = {"__step__": torch.tensor([self.step_count], dtype=torch.float32)}
        m, v = self.flat.full_moments()
        for name, p, o, n in self.flat.entries:
            out["m." + name] = m[o:o + n].view(p.shape)
            out["v." + name] = v[o:o + n].view(p.shape)
        return out

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        if "__step__" in sd:
            self.step_count = int(sd["__step__"].item())
        for name, p, o, n in self.flat.entries:
            if "m." + name in sd:
                self.flat.load_moments(name, sd["m." + name], sd["v." + name])
