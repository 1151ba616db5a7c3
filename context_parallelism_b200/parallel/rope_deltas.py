"""RoPE position deltas for one ring step (the reference's "4-delta" scheme).

The reference's fused kernel masks causally on *local* indices only and receives the global
RoPE position of a local row through two pairs of offsets, one pair per operand: ``d0`` applies
to the first half of the passed tensor and ``d1`` to the second half
(context_parallel/RopeDeltas.h:26-87).  The B200 kernels in this package take explicit per-tile
global positions instead, but the delta table remains the contract for the NCCL-rotator
baseline path and is checked against the reference's golden table
(Tests/cp_rope_deltas_test.cpp:58-84).
"""
from __future__ import annotations

import enum
from typing import NamedTuple


class SubChunk(enum.Enum):
    """Which operand was cut to one half this ring step (RopeDeltas.h:36-40)."""
    Full = 0        # step 0: full [head|tail] Q against full [head|tail] K, causal
    KHeadHalf = 1   # 0 < i <= rank: full Q against K[:Tl/2] (head half of the source)
    QTailHalf = 2   # i > rank: Q[Tl/2:] (tail half) against full K


class Deltas(NamedTuple):
    d0: int
    d1: int


class SdpaDeltas(NamedTuple):
    q: Deltas
    k: Deltas


def rope_source_rank(r: int, i: int, n: int) -> int:
    """Owner of the K/V block that rank ``r`` consumes at ring step ``i``."""
    return (r - i) % n


def rope_global_pos(j: int, length: int, d: Deltas) -> int:
    return j + (d.d1 if j >= length // 2 else d.d0)


def subchunk_for_step(r: int, i: int, load_balance: bool) -> SubChunk:
    """Sub-chunk rule of the HeadTail ring (ContextParallel.h:753-784)."""
    if not load_balance or i == 0:
        return SubChunk.Full
    return SubChunk.KHeadHalf if i <= r else SubChunk.QTailHalf


def compute_deltas(r: int, i: int, n: int, tl: int, lb: bool, sc: SubChunk) -> SdpaDeltas:
    s = rope_source_rank(r, i, n)
    if not lb:
        return SdpaDeltas(Deltas(r * tl, r * tl), Deltas(s * tl, s * tl))
    cs = tl // 2
    head = lambda x: x * cs
    tail = lambda x: (2 * n - 1 - x) * cs
    q = Deltas(head(r), tail(r) - cs)
    k = Deltas(head(s), tail(s) - cs)
    if sc is SubChunk.KHeadHalf:
        k = Deltas(head(s), head(s))
    elif sc is SubChunk.QTailHalf:
        q = Deltas(tail(r), tail(r))
    return SdpaDeltas(q, k)
