"""Sequence-axis gathers: HeadTail load-balance / unload-balance, local-shard gather of token ids and
activations, K/V packing.  One vectorised (16-byte) kernel serves every dtype
(``gather_seq_kernel``); replaces context_parallel/headtail_kernel.cu:26-105 (fp32 only, one element
per thread, plus a temp copy and a stream synchronise in context_parallel/ContextParallel.cpp:117-128)
and context_parallel/KVPackKernel.cu:13-37.
"""
from __future__ import annotations

import torch

from .. import _native as nv
from ..parallel import shard


def gather_seq(x: torch.Tensor, index: torch.Tensor, dim: int = 1) -> torch.Tensor:
    """``out = x.index_select(dim, index)``."""
    index = index.to(device=x.device, dtype=torch.int64).contiguous()
    if not x.is_cuda:
        return x.index_select(dim, index)
    x = x.contiguous()
    outer = 1
    for s in x.shape[:dim]:
        outer *= s
    inner = x.element_size()
    for s in x.shape[dim + 1:]:
        inner *= s
    out = torch.empty(x.shape[:dim] + (index.numel(),) + x.shape[dim + 1:], dtype=x.dtype, device=x.device)
    st = nv.status_for(x.device)
    nv.call("gather_seq", nv.ptr(x), nv.ptr(out), nv.ptr(index), nv.l(outer), nv.l(x.shape[dim]), nv.l(index.numel()),
            nv.l(inner), st.ptr(), nv.stream_ptr(x.device))
    return out


def gather_tokens(idx: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """Local shard of ``[B, T]`` token ids / targets at global positions ``pos``."""
    return gather_seq(idx, pos, dim=1)


def headtail_loadbalance(x: torch.Tensor, n: int, dim: int = 1) -> torch.Tensor:
    """Reorder the sequence axis so that rank r's HeadTail shard is the contiguous slice r
    (``HeadTail::loadbalance``, context_parallel/LoadBalancer.h:40-50)."""
    return gather_seq(x, shard.headtail_perm(x.shape[dim], n), dim)


def headtail_unloadbalance(x: torch.Tensor, n: int, dim: int = 1) -> torch.Tensor:
    return gather_seq(x, shard.headtail_inverse_perm(x.shape[dim], n), dim)


def kv_pack(k: torch.Tensor, v: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """Strided ``[B,T,H,D]`` K and V views → one contiguous ``[2,B,T,H,D]`` buffer (the message of one
    ring hop)."""
    B, T, H, D = k.shape
    if not k.is_cuda:
        return torch.stack([k, v]).contiguous()
    ok = lambda t: t.stride(3) == 1 and t.stride(2) == D and t.stride(0) == T * t.stride(1)
    if not (ok(k) and ok(v)):
        k, v = k.contiguous(), v.contiguous()
    if out is None:
        out = torch.empty((2, B, T, H, D), dtype=k.dtype, device=k.device)
    nv.call("kv_pack", nv.ptr(k), nv.ptr(v), nv.ptr(out), nv.l(B * T), nv.i(H * D), nv.l(k.stride(1)), nv.l(v.stride(1)),
            nv.stream_ptr(k.device))
    return out
