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


def parse_longrope_factors(path: str):
    """LongRoPE factors file: ``key=value`` header lines (``n_hat``, ``s``, ``search_len``) and one line of
    whitespace/comma separated λ values (``lambda=...`` or bare).  Returns ``(lam, n_hat, s, search_len)``."""
    lam, n_hat, s, slen = None, 0, 0, 0
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#"):
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
                lam = [float(t) for t in line.replace(",", " ").split()]
    if lam is None:
        raise ValueError(f"{path}: no lambda vector found")
    return lam, n_hat, s, slen
