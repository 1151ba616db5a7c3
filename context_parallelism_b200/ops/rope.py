"""RoPE cos/sin caches: plain, YaRN (NTK-by-parts + temperature) and LongRoPE (searched per-dimension
rescale λ with an initial-token threshold n̂), plus CREAM-style row gathers.

The reference builds these tables with CPU loops and copies them over
(context_parallel/YARNOps.cpp:49-138,150-208); here the table is produced on the device by
``rope_cache_kernel`` from a tiny per-dimension frequency vector prepared on the host.  Table layout:
``[seq_len, head_dim]`` fp32, row ``p`` = ``[cos(p·f_i)·m | sin(p·f_i)·m]`` (NeoX half-split).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import _native as nv
from ..config import YarnConfig
from . import reference as ref


def build_rope_cache(seq_len: int, head_dim: int, base: float, device, yarn: Optional[YarnConfig] = None,
                     positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    yarn = yarn or YarnConfig()
    device = torch.device(device)
    if device.type != "cuda":
        return ref.build_rope_cache(seq_len, head_dim, base, yarn.scale, yarn.orig_maxpos, yarn.beta_fast,
                                    yarn.beta_slow, yarn.no_mscale, positions)
    inv, _, _ = ref.yarn_inv_freq(head_dim, base, yarn.scale, yarn.orig_maxpos, yarn.beta_fast, yarn.beta_slow)
    m = ref.yarn_mscale(yarn.scale, yarn.no_mscale)
    inv = inv.to(device)
    n = seq_len if positions is None else positions.numel()
    cache = torch.empty((n, head_dim), dtype=torch.float32, device=device)
    pos = positions.to(device=device, dtype=torch.int64).contiguous() if positions is not None else None
    nv.call("rope_cache", nv.ptr(cache), nv.ptr(inv), nv.ptr(None), nv.ptr(pos), nv.l(n), nv.i(head_dim // 2),
            nv.l(0), nv.f(m), nv.stream_ptr(device))
    return cache


def build_rope_cache_longrope(seq_len: int, head_dim: int, base: float, lam: Sequence[float], n_hat: int,
                              device, mscale: float = 1.0) -> torch.Tensor:
    ref.validate_longrope(lam, head_dim, n_hat)
    device = torch.device(device)
    if device.type != "cuda":
        return ref.build_rope_cache_longrope(seq_len, head_dim, base, lam, n_hat, mscale)
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    base_freq = (1.0 / torch.pow(torch.tensor(float(base)), 2.0 * i / head_dim)).to(device)
    lam_t = torch.tensor(list(lam), dtype=torch.float32, device=device)
    cache = torch.empty((seq_len, head_dim), dtype=torch.float32, device=device)
    nv.call("rope_cache", nv.ptr(cache), nv.ptr(base_freq), nv.ptr(lam_t), nv.ptr(None), nv.l(seq_len), nv.i(half),
            nv.l(n_hat), nv.f(mscale), nv.stream_ptr(device))
    return cache


def gather_cache_rows(cache: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """``cache[labels]`` — installs CREAM / PoSE / RandPos position labels
    (Scripts/Blutrain/bluscriptCP.cpp:467-494)."""
    labels = labels.to(device=cache.device, dtype=torch.int64).contiguous()
    if not cache.is_cuda:
        return cache[labels].contiguous()
    out = torch.empty((labels.numel(), cache.shape[1]), dtype=torch.float32, device=cache.device)
    st = nv.status_for(cache.device)
    nv.call("gather_rows_f32", nv.ptr(cache), nv.ptr(labels), nv.ptr(out), nv.l(labels.numel()), nv.i(cache.shape[1]),
            nv.l(cache.shape[0]), st.ptr(), nv.stream_ptr(cache.device))
    return out


def parse_longrope_factors(path: str, half: int = 0):
    """LongRoPE factors file in the reference's layout (Scripts/Blutrain/bluscriptCP.cpp:538-572): whitespace
    separated tokens, keys in any order,

        n_hat <int>
        s <int>                extension ratio the search used
        S_search <int>         target length of the search
        lambda <f0> <f1> ...   head_dim/2 non-decreasing values >= 1

    a token starting with ``#`` comments out the rest of its line.  Also accepted, for files written by earlier
    versions of this package: ``key=value`` header lines with a bare line of λ values.  ``half`` (head_dim / 2), when
    given, is the exact number of λ values required.  Returns ``(lam, n_hat, s, search_len)``; raises ``ValueError``
    on any malformation (missing ``n_hat``, too few values, a value below 1, a decreasing value)."""
    with open(path) as f:
        text = f.read()
    lam, n_hat, s, slen = None, -1, -1, -1
    lines = [ln.split("#", 1)[0] for ln in text.splitlines()]
    if any("=" in ln for ln in lines):
        for line in lines:
            line = line.strip()
            if not line:
                continue
            if "=" in line:
                k, v = line.split("=", 1)
                k = k.strip().lower()
                if k in ("n_hat", "nhat"):
                    n_hat = int(float(v))
                elif k == "s":
                    s = int(float(v))
                elif k in ("search_len", "s_search"):
                    slen = int(float(v))
                elif k in ("lambda", "factors"):
                    lam = [float(t) for t in v.replace(",", " ").split()]
                else:
                    raise ValueError(f"{path}: unexpected key {k!r}")
            else:
                lam = [float(t) for t in line.replace(",", " ").split()]
    else:
        toks = " ".join(lines).split()
        i = 0

        def number(kind, what):
            nonlocal i
            i += 1
            if i >= len(toks):
                raise ValueError(f"{path}: bad {what}")
            try:
                return kind(toks[i])
            except ValueError:
                raise ValueError(f"{path}: bad {what}") from None
        while i < len(toks):
            t = toks[i]
            if t == "n_hat":
                n_hat = number(int, "n_hat")
            elif t == "s":
                s = number(int, "s")
            elif t == "S_search":
                slen = number(int, "S_search")
            elif t == "lambda":
                lam = []
                while i + 1 < len(toks) and (half <= 0 or len(lam) < half):
                    try:
                        lam.append(float(toks[i + 1]))
                    except ValueError:
                        break
                    i += 1
            else:
                raise ValueError(f"{path}: unexpected token {t!r}")
            i += 1
    if not lam:
        raise ValueError(f"{path}: missing 'lambda'")
    if half > 0 and len(lam) != half:
        raise ValueError(f"{path}: expected {half} lambda values, found {len(lam)}")
    if n_hat < 0:
        raise ValueError(f"{path}: missing 'n_hat'")
    for j, v in enumerate(lam):
        if not v >= 1.0:
            raise ValueError(f"{path}: lambda must be >= 1")
        if j > 0 and v < lam[j - 1]:
            raise ValueError(f"{path}: lambda must be non-decreasing")
    return lam, n_hat, max(s, 0), max(slen, 0)


def write_longrope_factors(path: str, lam, n_hat: int, s: float, search_len: int) -> None:
    """Write a factors file the reference's trainer reads (``n_hat`` / ``s`` / ``S_search`` / ``lambda`` tokens), atomically."""
    import os
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        f.write(f"n_hat {int(n_hat)}\ns {int(s)}\nS_search {int(search_len)}\nlambda " + " ".join(f"{float(v):.6f}" for v in lam) + "\n")
    os.replace(tmp, path)
