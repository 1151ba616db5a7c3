"""Learning-rate schedules: linear warm-up + cosine decay to ``min_lr``
(Scripts/Blutrain/gpt2_cp_test.cpp:1680; bluscriptCP.cpp:518-531) and the two-stage re-warm-up used when
a run resumes for context extension (bluscriptCP.cpp:1204-1221: a fresh ramp anchored at the resume
step, optionally to a reduced peak)."""
from __future__ import annotations

import math


def cosine_lr(step: int, max_lr: float, min_lr: float, warmup: int, max_steps: int) -> float:
    if step < warmup:
        return max_lr * (step + 1) / max(1, warmup)
    if step >= max_steps:
        return min_lr
    ratio = (step - warmup) / max(1, max_steps - warmup)
    return min_lr + 0.5 * (1.0 + math.cos(math.pi * ratio)) * (max_lr - min_lr)


def rewarmup_lr(step: int, max_lr: float, min_lr: float, warmup: int, max_steps: int,
                anchor: int, rewarmup: int, peak_frac: float = 1.0) -> float:
    """Schedule for a resumed run: for ``anchor <= step < anchor+rewarmup`` ramp linearly from 0 to the value
    the (peak-scaled) cosine schedule has at the end of the ramp; afterwards follow that schedule."""
    if rewarmup <= 0 or anchor < 0 or step < anchor:
        return cosine_lr(step, max_lr, min_lr, warmup, max_steps)
    peak = max_lr * peak_frac
    base = lambda s: cosine_lr(s, peak, min(min_lr, peak), warmup, max_steps)
    if step < anchor + rewarmup:
        return base(anchor + rewarmup) * (step - anchor + 1) / rewarmup
    return base(step)
