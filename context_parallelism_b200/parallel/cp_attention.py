"""Context-parallel attention layer: one entry point for every mode.

``CPAttention(qkv, pos)`` takes the packed, already normalised and rotated projections of the LOCAL
tokens ``[B, T_local, (Hq + 2·Hkv)·D]`` with their global positions and returns ``[B, T_local, Hq·D]``.
Modes (``CP_ATTN_MODE``): ``ring`` (HeadTail load-balanced), ``ulysses`` (contiguous shards, head
all-to-all), ``hybrid`` (Ulysses inside, ring outside).  Transport (``CP_ROTATOR``): ``fused`` uses the
peer-memory kernels of this package; ``p2p`` / ``alltoall`` / ``allgather`` select the NCCL-only
baseline built on ``torch.distributed``.  This mirrors the dispatch of
``ContextParallel::forward_cp`` (context_parallel/ContextParallel.h:405-422,1359-1396) with
``pre_sharded=true, unshard=false``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist

from ..config import Config
from ..ops import attention as A
from . import shard
from .mesh import DeviceMesh


@dataclass
class CPContext:
    cfg: Config
    mesh: Optional[DeviceMesh] = None
    cp_group: object = None
    cp_rank: int = 0
    cp_size: int = 1
    ring_group: object = None
    ring_rank: int = 0
    ring_size: int = 1
    ulysses_group: object = None
    ulysses_rank: int = 0
    ulysses_size: int = 1
    dp_rank: int = 0
    dp_size: int = 1
    world_group: object = None
    fused: object = None            # parallel.fused.FusedComm once initialised (CUDA, same node)

    @staticmethod
    def single(cfg: Config) -> "CPContext":
        return CPContext(cfg=cfg)

    @staticmethod
    def from_mesh(cfg: Config, mesh: DeviceMesh) -> "CPContext":
        c = CPContext(cfg=cfg, mesh=mesh, world_group=None)
        c.dp_rank, c.dp_size = mesh.coord("dp"), mesh.size("dp")
        if cfg.attn_mode == "hybrid":
            c.ring_group, c.ring_rank, c.ring_size = mesh.group("ring"), mesh.coord("ring"), mesh.size("ring")
            c.ulysses_group, c.ulysses_rank, c.ulysses_size = mesh.group("ulysses"), mesh.coord("ulysses"), mesh.size("ulysses")
            c.cp_size = c.ring_size * c.ulysses_size
            c.cp_rank = c.ring_rank * c.ulysses_size + c.ulysses_rank
        else:
            c.cp_group, c.cp_rank, c.cp_size = mesh.group("cp"), mesh.coord("cp"), mesh.size("cp")
            if cfg.attn_mode == "ring":
                c.ring_group, c.ring_rank, c.ring_size = c.cp_group, c.cp_rank, c.cp_size
            else:
                c.ulysses_group, c.ulysses_rank, c.ulysses_size = c.cp_group, c.cp_rank, c.cp_size
        return c

    # ------------------------------------------------------------------ sharding of a batch
    def local_positions(self, T: int) -> torch.Tensor:
        cfg = self.cfg
        if self.cp_size == 1:
            return torch.arange(T)
        if cfg.attn_mode == "hybrid":
            return shard.hybrid_local_positions(T, self.ring_size, self.ring_rank, self.ulysses_size, self.ulysses_rank)
        return shard.local_positions(T, self.cp_size, self.cp_rank, cfg.load_balance)

    def ring_positions(self, T: int) -> List[torch.Tensor]:
        """Position vectors of every ring rank's block (after the Ulysses combine in hybrid mode)."""
        lb = self.cfg.load_balance or self.cfg.attn_mode == "hybrid"
        return [shard.local_positions(T, self.ring_size, s, lb) for s in range(self.ring_size)]


class _ShardSeq(torch.autograd.Function):
    """Full sequence ``[B, T, ...]`` (the same tensor on every rank of the group) -> this rank's tokens; the adjoint
    gathers every rank's gradient block and puts it back at its positions, so each rank ends with the full-sequence
    gradient (the internal sharding of ``forward_cp(pre_sharded=false)`` and its three backward all-gathers,
    context_parallel/ContextParallel.h:467-495, context_parallel/ContextParallelBackward.h:781-813)."""

    @staticmethod
    def forward(ctx, x, all_pos, rank, group):
        ctx.all_pos, ctx.group, ctx.T = all_pos, group, x.shape[1]
        return x.index_select(1, all_pos[rank].to(x.device)).contiguous()

    @staticmethod
    def backward(ctx, g):
        return _gather_seq(g.contiguous(), ctx.all_pos, ctx.group, ctx.T), None, None, None


class _UnshardSeq(torch.autograd.Function):
    """This rank's tokens -> the full sequence on every rank (all-gather + un-permute: ``forward_cp(unshard=true)``,
    ContextParallel.h:1159-1203; UlyssesAttention.h:104-131); the adjoint keeps the local rows of the gradient."""

    @staticmethod
    def forward(ctx, x, all_pos, rank, group):
        ctx.pos = all_pos[rank]
        return _gather_seq(x.contiguous(), all_pos, group, sum(int(p.numel()) for p in all_pos))

    @staticmethod
    def backward(ctx, g):
        return g.index_select(1, ctx.pos.to(g.device)).contiguous(), None, None, None


def _gather_seq(x: torch.Tensor, all_pos, group, T: int) -> torch.Tensor:
    n = len(all_pos)
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x, group=group)
    full = torch.empty((x.shape[0], T) + tuple(x.shape[2:]), dtype=x.dtype, device=x.device)
    for r in range(n):
        full.index_copy_(1, all_pos[r].to(x.device), parts[r])
    return full


class CPAttention:
    def __init__(self, cfg: Config, ctx: CPContext):
        self.cfg, self.ctx = cfg, ctx
        self.scale = cfg.head_dim ** -0.5
        self._pos_cache = {}
        from ..utils.debug import DebugTools
        rank = dist.get_rank() if dist.is_initialized() else 0
        self.dbg = ctx.fused.dbg if ctx.fused is not None else DebugTools(cfg, rank)

    def _ring_pos(self, T: int, device):
        key = (T, str(device))
        v = self._pos_cache.get(key)
        if v is None:
            allp = self.ctx.ring_positions(T)
            v = (allp, allp[self.ctx.ring_rank].to(device))
            self._pos_cache[key] = v
        return v

    def forward_cp(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, unshard: bool = False,
                   pre_sharded: bool = True) -> torch.Tensor:
        """``ContextParallel::forward_cp(q, k, v, unshard, pre_sharded)`` (context_parallel/ContextParallel.h:405-409)
        on token-major tensors ``[B, T, H, D]``.  ``pre_sharded=False``: q/k/v hold the FULL sequence on every rank and
        are sharded here (HeadTail for ring / hybrid, contiguous for Ulysses); ``unshard=True``: the result is gathered
        back to the full sequence on every rank.  Both are differentiable.  The trainers use
        ``pre_sharded=True, unshard=False`` (``__call__``)."""
        ctx = self.ctx
        if ctx.cp_size == 1:
            return self._attend(q, k, v)
        if pre_sharded and not unshard:
            return self._attend(q, k, v)
        if ctx.cfg.attn_mode == "hybrid":
            raise ValueError("forward_cp with internal sharding / unsharding is provided for ring and ulysses")
        T = q.shape[1] if not pre_sharded else q.shape[1] * ctx.cp_size
        all_pos = [_at_rank(ctx, r).local_positions(T) for r in range(ctx.cp_size)]
        group = ctx.cp_group
        if not pre_sharded:
            q, k, v = (_ShardSeq.apply(t, all_pos, ctx.cp_rank, group) for t in (q, k, v))
        o = self._attend(q, k, v)
        if unshard:
            o = _UnshardSeq.apply(o, all_pos, ctx.cp_rank, group)
        return o

    def __call__(self, qkv: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        B, Tl = qkv.shape[:2]
        Hq, Hkv, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
        x = qkv.view(B, Tl, Hq + 2 * Hkv, D)
        q, k, v = x[:, :, :Hq], x[:, :, Hq:Hq + Hkv], x[:, :, Hq + Hkv:]
        return self._attend(q, k, v).reshape(B, Tl, Hq * D)

    def _attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """Attention over the local tokens ``[B, T_local, H, D]`` in the configured mode."""
        cfg, ctx = self.cfg, self.ctx
        qkv = q
        B, Tl = q.shape[:2]
        Hq, Hkv, D = q.shape[2], k.shape[2], q.shape[3]
        mode = cfg.attn_mode if ctx.cp_size > 1 else "single"
        fused = ctx.fused is not None and cfg.rotator == "fused" and qkv.is_cuda
        if mode == "single":
            o, _ = A.flash_attention(q, k, v, self.scale, True)
        elif mode == "ring":
            T = Tl * ctx.ring_size
            allp, mypos = self._ring_pos(T, qkv.device)
            if fused:
                o = ctx.fused.ring_attention(q, k, v, mypos, T, self.scale)
            else:
                from .ring import ring_attention
                kind = "p2p" if cfg.rotator == "fused" else cfg.rotator
                # the reference keeps the N-1 received K/V blocks for backward unless CP_RECOMPUTE_K asks to rotate
                # them again (context_parallel/ContextParallelBackward.h:214-242)
                o, _ = ring_attention(q, k, v, mypos, allp, ctx.ring_group, kind, self.scale, not cfg.recompute_k, self.dbg)
        elif mode == "ulysses":
            if fused:
                o = ctx.fused.ulysses_attention(q, k, v, self.scale)
            else:
                from .ulysses import ulysses_attention
                o = ulysses_attention(q, k, v, ctx.ulysses_group, self.scale)
        elif mode == "hybrid":
            from .hybrid import hybrid_attention
            o = hybrid_attention(q, k, v, ctx, self, fused)
        else:
            raise ValueError(mode)
        return o


def _at_rank(ctx: CPContext, r: int) -> CPContext:
    """A copy of the context as cp rank ``r`` sees it (for position tables of the other ranks)."""
    import dataclasses
    return dataclasses.replace(ctx, cp_rank=r, ring_rank=r if ctx.cfg.attn_mode == "ring" else ctx.ring_rank,
                               ulysses_rank=r if ctx.cfg.attn_mode == "ulysses" else ctx.ulysses_rank)
