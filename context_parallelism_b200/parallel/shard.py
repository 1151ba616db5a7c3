"""Sequence sharding index math: contiguous, HeadTail (zig-zag) and hybrid.

HeadTail splits a length-T sequence into 2N equal chunks and gives rank r chunks
``(r, 2N-1-r)`` laid out ``[head | tail]`` so that every rank does the same amount of causal
work (context_parallel/ContextParallel.h:102-139; permutation example N=2,T=8 →
``[0,1,6,7,2,3,4,5]``, context_parallel/headtail_kernel.cuh:12-13).  The hybrid layout applies
HeadTail over the ring axis and then a contiguous split over the Ulysses axis
(ContextParallel.h:194-228).

All builders are pure index math, cached per ``(T, mesh coordinates)``; the gather itself is
one device kernel per batch (``ops.permute``).
"""
from __future__ import annotations

import functools
from typing import Optional, Tuple

import torch


def headtail_perm(T: int, n: int) -> torch.Tensor:
    """Full-sequence permutation: ``out[j] = x[perm[j]]`` puts rank r's shard at
    ``[r*T/n, (r+1)*T/n)`` (the layout ``HeadTail::loadbalance`` produces,
    context_parallel/LoadBalancer.h:40-50)."""
    if T % (2 * n):
        raise ValueError(f"HeadTail needs T={T} divisible by 2*N={2 * n}")
    cs = T // (2 * n)
    chunks = []
    for r in range(n):
        chunks.append(torch.arange(r * cs, (r + 1) * cs))
        chunks.append(torch.arange((2 * n - 1 - r) * cs, (2 * n - r) * cs))
    return torch.cat(chunks)


def headtail_inverse_perm(T: int, n: int) -> torch.Tensor:
    """Permutation that undoes :func:`headtail_perm` (``HeadTail::unloadbalance``)."""
    p = headtail_perm(T, n)
    inv = torch.empty_like(p)
    inv[p] = torch.arange(T)
    return inv


@functools.lru_cache(maxsize=256)
def _local_positions_cached(T: int, n: int, rank: int, load_balance: bool) -> torch.Tensor:
    tl = T // n
    if not load_balance:
        return torch.arange(rank * tl, (rank + 1) * tl)
    if T % (2 * n):
        raise ValueError(f"HeadTail needs T={T} divisible by 2*N={2 * n}")
    cs = T // (2 * n)
    return torch.cat([torch.arange(rank * cs, (rank + 1) * cs),
                      torch.arange((2 * n - 1 - rank) * cs, (2 * n - rank) * cs)])


def local_positions(T: int, n: int, rank: int, load_balance: bool) -> torch.Tensor:
    """Global positions (int64, CPU) of rank ``rank``'s local tokens, in local order."""
    if T % n:
        raise ValueError(f"T={T} % N={n} != 0")
    return _local_positions_cached(T, n, rank, load_balance)


@functools.lru_cache(maxsize=256)
def _hybrid_positions_cached(T: int, r_size: int, r_rank: int, u_size: int, u_rank: int) -> torch.Tensor:
    ring_block = _local_positions_cached(T, r_size, r_rank, True)
    t_ring = T // r_size
    if t_ring % u_size:
        raise ValueError("hybrid: T/ring_size must be divisible by ulysses_size")
    tl = t_ring // u_size
    return ring_block[u_rank * tl:(u_rank + 1) * tl].clone()


def hybrid_local_positions(T: int, ring_size: int, ring_rank: int,
                           ulysses_size: int, ulysses_rank: int) -> torch.Tensor:
    """HeadTail over the ring axis, then contiguous piece ``ulysses_rank`` of that ring block."""
    if T % (2 * ring_size):
        raise ValueError("hybrid: T must be divisible by 2*ring_size (HeadTail)")
    return _hybrid_positions_cached(T, ring_size, ring_rank, ulysses_size, ulysses_rank)


def local_to_global_pos(rank: int, i: int, tl: int, n: int, load_balance: bool) -> int:
    """Scalar form of :func:`local_positions` (context_parallel/RopeDeltas.h:96-101)."""
    if not load_balance:
        return rank * tl + i
    cs = tl // 2
    return rank * cs + i if i < cs else (2 * n - 1 - rank) * cs + (i - cs)


def shard_sequence_pre_embed(idx: torch.Tensor, targets: Optional[torch.Tensor], T: int, n: int,
                             rank: int, load_balance: bool
                             ) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor]:
    """Gather the local token ids / targets and return them with their global positions.

    ``idx``/``targets`` are ``[B, T]``; the result is ``([B, T/n], [B, T/n] | None, [T/n] int64)``.
    Targets must be sharded with the identical permutation as the inputs
    (Scripts/Blutrain/bluscriptCP.cpp:1230-1236)."""
    pos = local_positions(T, n, rank, load_balance).to(idx.device)
    from ..ops import permute
    idx_l = permute.gather_tokens(idx, pos)
    tgt_l = permute.gather_tokens(targets, pos) if targets is not None else None
    return idx_l, tgt_l, pos


def shard_sequence_pre_embed_hybrid(idx, targets, T, ring_size, ring_rank, ulysses_size, ulysses_rank):
    pos = hybrid_local_positions(T, ring_size, ring_rank, ulysses_size, ulysses_rank).to(idx.device)
    from ..ops import permute
    idx_l = permute.gather_tokens(idx, pos)
    tgt_l = permute.gather_tokens(targets, pos) if targets is not None else None
    return idx_l, tgt_l, pos


def chunk_owner(chunk: int, n: int) -> int:
    """Rank that owns HeadTail chunk ``chunk`` of the 2N chunks."""
    return chunk if chunk < n else 2 * n - 1 - chunk
