"""DeepSpeed-Ulysses sequence↔head all-to-all on ``torch.distributed`` — the NCCL-only baseline.

``seq_to_head``: ``[B, T/P, H, D] → [B, T, H/P, D]`` and ``head_to_seq`` its inverse; the two are each
other's adjoint, so each one's backward is the other (context_parallel/UlyssesAttention.h:43-97,
context_parallel/UlyssesAttentionBackward.h).  GQA with fewer KV heads than ranks replicates KV heads
``P/Hkv`` times before the exchange and sums the replicas' gradients afterwards
(``head_repeat_interleave`` / ``head_group_reduce``, UlyssesAttention.h:143-169;
ContextParallel.h:1517-1548).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import attention as A


def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x, group=group)
    return out


class _SeqToHead(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        P = dist.get_world_size(group)
        B, Tl, H, D = x.shape
        Hl = H // P
        send = x.view(B, Tl, P, Hl, D).permute(2, 0, 1, 3, 4).contiguous()          # [P,B,Tl,Hl,D]
        recv = _a2a(send, group)                                                     # chunk p = tokens of rank p
        return recv.permute(1, 0, 2, 3, 4).reshape(B, P * Tl, Hl, D)

    @staticmethod
    def backward(ctx, g):
        return _HeadToSeq.apply(g.contiguous(), ctx.group), None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        P = dist.get_world_size(group)
        B, T, Hl, D = x.shape
        Tl = T // P
        send = x.view(B, P, Tl, Hl, D).permute(1, 0, 2, 3, 4).contiguous()          # [P,B,Tl,Hl,D]
        recv = _a2a(send, group)                                                     # chunk p = heads of rank p
        return recv.permute(1, 2, 0, 3, 4).reshape(B, Tl, P * Hl, D)

    @staticmethod
    def backward(ctx, g):
        return _SeqToHead.apply(g.contiguous(), ctx.group), None


def seq_to_head(x: torch.Tensor, group) -> torch.Tensor:
    return _SeqToHead.apply(x.contiguous(), group)


def head_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    return _HeadToSeq.apply(x.contiguous(), group)


def kv_replication(n_kv: int, P: int) -> int:
    if n_kv % P == 0:
        return 1
    if P % n_kv == 0:
        return P // n_kv
    raise ValueError(f"ulysses: kv_heads={n_kv} and P={P} must divide one another")


def ulysses_attention(q, k, v, group, scale: Optional[float] = None):
    """q ``[B,Tl,Hq,D]``, k/v ``[B,Tl,Hkv,D]`` sharded contiguously over ``group`` → ``[B,Tl,Hq,D]``."""
    P = dist.get_world_size(group)
    Hq, Hkv = q.shape[2], k.shape[2]
    if Hq % P:
        raise ValueError(f"ulysses: q_heads={Hq} % P={P} != 0")
    rep = kv_replication(Hkv, P)
    if rep > 1:
        idx = torch.arange(Hkv * rep, device=k.device) // rep
        k, v = k.index_select(2, idx), v.index_select(2, idx)
    qh, kh, vh = seq_to_head(q, group), seq_to_head(k, group), seq_to_head(v, group)
    o, _ = A.flash_attention(qh, kh, vh, scale, True)
    return head_to_seq(o, group)
