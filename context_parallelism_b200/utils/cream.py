"""Position-label generators for context-window extension: CREAM, PoSE and RandPos.

A label vector ``L`` of length T assigns an absolute RoPE position to each physical token;
gathering the cos/sin cache rows at ``L`` makes the model rotate at larger positions while the
attention matrix stays T×T (context_parallel/CreamPositions.h:41-221; installed by a row
gather of the cache, Scripts/Blutrain/bluscriptCP.cpp:467-494).

Numerical hazards the generators must respect (CreamPositions.h:11-20): the truncated-Gaussian
factor is *truncated* to int, ``rand_factor/2`` is a true division, and random integer draws
are inclusive at both ends.  The deterministic layers are tested against the reference's
golden tuples (Tests/cream_positions_test.cpp:48-90); the random stream itself is ours.
"""
from __future__ import annotations

import math
import random
from typing import List, Tuple

import numpy as np


def cream_head_tail_len(T: int, factor: int, branch: int) -> int:
    return T // 3 if branch == 0 else 4 * factor


def cream_validate(T: int, factor: int, branch: int) -> None:
    if factor < 2:
        raise ValueError(f"cream: factor(=YARN_SCALE) must be >= 2, got {factor}")
    ht = cream_head_tail_len(T, factor, branch)
    if 2 * ht >= T:
        raise ValueError(f"cream: head+tail(={2 * ht}) >= T(={T}) -- degenerate middle")


def cream_labels_from_draws(T: int, factor: int, branch: int, rand_factor: int, end_id: int) -> List[int]:
    """``[0,head) ++ [end_id-(len_chunk-1), end_id] ++ [factor*T-tail, factor*T)``."""
    cream_validate(T, factor, branch)
    ht = cream_head_tail_len(T, factor, branch)
    len_chunk = T - 2 * ht
    smax = factor * T
    return (list(range(ht)) + list(range(end_id - (len_chunk - 1), end_id + 1))
            + list(range(smax - ht, smax)))


def rand_factor_from_u(u: float, factor: int, sigma: float) -> int:
    """Inverse CDF of a Gaussian(μ=1+factor, σ) tabulated on ``linspace(2, 2·factor, 1000)``;
    the interpolated value is truncated toward zero."""
    mu = 1.0 + factor
    x = np.linspace(2.0, 2.0 * factor, 1000)
    cdf = np.array([0.5 * (1.0 + math.erf((xi - mu) / (sigma * math.sqrt(2.0)))) for xi in x])
    rf = int(np.interp(u, cdf, x))
    return max(2, min(2 * factor, rf))


def end_id_range(T: int, factor: int, branch: int, rand_factor: int) -> Tuple[int, int]:
    ht = cream_head_tail_len(T, factor, branch)
    len_chunk = T - 2 * ht
    half = rand_factor / 2.0
    lo = int(ht + (len_chunk - 1) * half)
    hi = int(round(half * T - ht - 1))
    return lo, hi


def generate_cream_positions(T: int, factor: int, sigma: float, seed: int) -> List[int]:
    rng = random.Random(seed)
    branch = rng.randint(0, 1)
    cream_validate(T, factor, branch)
    rf = rand_factor_from_u(rng.random(), factor, sigma)
    lo, hi = end_id_range(T, factor, branch, rf)
    end_id = rng.randint(lo, max(lo, hi))
    return cream_labels_from_draws(T, factor, branch, rf, end_id)


def generate_pose_positions(T: int, factor: int, seed: int) -> List[int]:
    """PoSE: ``[0, rt1) ++ (arange(rt1, T) + rt)`` with ``rt1∈[1,(T+1)//2]``, ``rt∈[0, factor·T−T]``."""
    if factor < 2:
        raise ValueError("pose: factor must be >= 2")
    rng = random.Random(seed)
    rt1 = rng.randint(1, (T + 1) // 2)
    rt = rng.randint(0, factor * T - T)
    return list(range(rt1)) + [j + rt for j in range(rt1, T)]


def generate_randpos_positions(T: int, factor: int, seed: int) -> List[int]:
    """RandPos: T distinct positions sampled from ``[0, factor·T)`` and sorted."""
    if factor < 2:
        raise ValueError("randpos: factor must be >= 2")
    rng = random.Random(seed)
    return sorted(rng.sample(range(factor * T), T))


def generate_positions(mode: str, T: int, factor: int, sigma: float, seed: int) -> List[int]:
    if mode == "cream":
        return generate_cream_positions(T, factor, sigma, seed)
    if mode == "pose":
        return generate_pose_positions(T, factor, seed)
    if mode == "randpos":
        return generate_randpos_positions(T, factor, seed)
    raise ValueError(f"unknown CP_CREAM_MODE {mode!r}")


def vhash(labels) -> int:
    """Order-sensitive checksum used by the golden tests: ``Σ (j+1)·L[j]``."""
    return int(sum((j + 1) * int(v) for j, v in enumerate(labels)))
