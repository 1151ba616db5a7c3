"""Hybrid (USP) attention: Ulysses all-to-all inside, ring outside.

The Ulysses combine over the inner group turns ``[B, T/(R·U), H, D]`` into ``[B, T/R, H/U, D]`` — the whole
HeadTail ring block of this ring rank with a slice of the heads — then ring attention runs over the
outer group and the result is partitioned back (context_parallel/ContextParallel.h:1359-1396,
context_parallel/HybridUlyssesBackward.h:42-81).  Requires ``q_heads % U == 0`` and ``kv_heads % U == 0``.  With the fused transport both the ring (copy CTAs inside the
attention kernel) and the Ulysses exchange (peer stores / pulls over the symmetric heap) run without NCCL.
"""
from __future__ import annotations

import os

import torch

from .ulysses import head_to_seq, seq_to_head


def hybrid_attention(q, k, v, ctx, attn, fused: bool):
    U, R = ctx.ulysses_size, ctx.ring_size
    if q.shape[2] % U or k.shape[2] % U:
        raise ValueError("hybrid: q_heads and kv_heads must be multiples of the Ulysses degree")
    # With the fused transport both axes go over peer memory: the sequence<->head exchange on the Ulysses axis around the
    # fused ring on the ring axis.  CP_FUSED_HYBRID_ULYSSES=0 keeps the NCCL all-to-all on the Ulysses axis.
    fused_uly = (fused and U > 1 and os.environ.get("CP_FUSED_HYBRID_ULYSSES", "1") == "1"
                 and getattr(ctx.fused, "g_uly", None) is not None and q.dtype == torch.bfloat16)
    ub = None
    dbg = getattr(attn, "dbg", None)
    if dbg is not None and dbg.d.selfcheck and U > 1 and not fused_uly:
        # CP_SELFCHECK in hybrid mode: the sequence<->head exchange must be an exact round trip
        # (context_parallel/ContextParallel.h:1307-1327)
        with torch.no_grad():
            back = head_to_seq(seq_to_head(q.detach().contiguous(), ctx.ulysses_group), ctx.ulysses_group)
        dbg.selfcheck("hybrid combine/partition round trip", dbg.next_call("hybrid"), {"q": q.detach()}, lambda: {"q": back})
    if fused_uly:
        from .fused import fused_head_to_seq, fused_seq_to_head
        q, k, v, ub = fused_seq_to_head(ctx.fused, q, k, v)
    elif U > 1:
        q, k, v = (seq_to_head(t, ctx.ulysses_group) for t in (q, k, v))
    T = q.shape[1] * R
    if R > 1:
        allp, mypos = attn._ring_pos(T, q.device)
        if fused and ctx.fused.supports_ring_group():
            o = ctx.fused.ring_attention(q, k, v, mypos, T, attn.scale)
        else:
            from .ring import ring_attention
            kind = "p2p" if attn.cfg.rotator == "fused" else attn.cfg.rotator
            o, _ = ring_attention(q, k, v, mypos, allp, ctx.ring_group, kind, attn.scale, not attn.cfg.recompute_k, attn.dbg)
    else:
        from ..ops import attention as A
        o, _ = A.flash_attention(q, k, v, attn.scale, True)
    if fused_uly:
        o = fused_head_to_seq(ctx.fused, o, ub)
    elif U > 1:
        o = head_to_seq(o, ctx.ulysses_group)
    return o
