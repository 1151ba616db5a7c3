"""Ring attention over a process group: the N-step K/V rotation with online-softmax merge and the
travelling dK/dV accumulator — the algorithm of the reference's ``ContextParallel::forward_cp`` and
``ContextParallelBackward`` (context_parallel/ContextParallel.h:507-1013,
context_parallel/ContextParallelBackward.h:275-716) — on ``torch.distributed`` rotators.

This is (a) the NCCL-only baseline the fused kernels are measured against and (b), on gloo/CPU with
the dense PyTorch attention, the end-to-end oracle.  Differences from the reference: masking uses
global positions, so each received block is processed as (up to) two position-contiguous halves with
the same kernel instead of the Full/KHeadHalf/QTailHalf case table, fully-masked tiles are skipped
inside the kernel, and nothing but the local K/V is saved for backward unless ``save_kv`` is set
(the reference saves all N received blocks unless ``CP_RECOMPUTE_K``).

Layout: q ``[B,Tl,Hq,D]``, k/v ``[B,Tl,Hkv,D]``; ``pos`` int64 ``[Tl]`` global positions (HeadTail or
contiguous).  K/V travel in bf16 on GPU (``CP_RING_BF16``) and dK/dV accumulate in fp32.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import attention as A
from ..ops import attention_bwd as AB
from ..ops import elementwise as E
from ..ops import reference as ref
from .rotators import make_rotator


def _halves(pos: torch.Tensor) -> List[Tuple[int, int, int]]:
    """Split a local position vector into maximal position-contiguous runs: ``(start_row, n_rows, first_pos)``."""
    p = pos.tolist()
    runs, s = [], 0
    for i in range(1, len(p) + 1):
        if i == len(p) or p[i] != p[i - 1] + 1:
            runs.append((s, i - s, p[s]))
            s = i
    return runs


def _fwd_block(q, kb, vb, scale, q_pos, k_off):
    if q.is_cuda:
        return A.flash_fwd(q, kb, vb, scale, True, q_pos.int(), k_off)
    kp = torch.arange(k_off, k_off + kb.shape[1])
    return ref.attention_dense(q, kb, vb, scale, q_pos, kp, True)


class _RingAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, pos, all_pos, group, rotator_kind, scale, save_kv, dbg):
        N, r = dist.get_world_size(group), dist.get_rank(group)
        B, Tl, Hq, D = q.shape
        kv = torch.stack([k, v]).contiguous()                      # [2,B,Tl,Hkv,D] message of one hop
        rot = make_rotator(rotator_kind, group)
        d = dbg.d if dbg is not None else None
        call = dbg.next_call("ring") if (dbg is not None and dbg.active) else 0
        blocking = d is not None and (d.ring_blocking or d.no_overlap or d.no_overlap_fwd or d.sync_ring)
        out = lse = None
        saved = []
        cur = kv
        for i in range(N):
            s = (r - i) % N
            handle = rot.exchange(cur) if i < N - 1 else None
            nxt = handle.wait() if (handle is not None and blocking) else None     # diagnostics: no look-ahead
            if blocking and q.is_cuda:
                torch.cuda.synchronize()
            if save_kv and i > 0:
                saved.append(cur)
            if dbg is not None:
                dbg.drain(1)
            for h, (row0, n, p0) in enumerate(_halves(all_pos[s])):
                ob, lb = _fwd_block(q, cur[0][:, row0:row0 + n], cur[1][:, row0:row0 + n], scale, pos, p0)
                if dbg is not None:
                    dbg.drain(2)
                    dbg.dump(d.dump_cp_steps, f"cp_step{i}_{h}", call, out=ob, lse=lb)
                if out is None:
                    out, lse = ob.clone(), lb.clone()
                else:
                    E.lse_merge_(out, lse, ob, lb)
                if dbg is not None:
                    dbg.drain(3)
                    dbg.dump(d.dump_cp_merge, f"cp_merge{i}_{h}", call, out=out, lse=lse)
            if handle is not None:
                cur = nxt if nxt is not None else handle.wait()
                if d is not None and d.fwd_sync_recv and q.is_cuda:
                    torch.cuda.synchronize()
        if dbg is not None and dbg.active:
            dbg.shapes("ring forward", q=q, kv=kv, out=out, lse=lse)
            dbg.dump(d.dump_cp_out, "cp_out", call, out=out, lse=lse)
            dbg.sync_if(d.fwd_sync_return)
        ctx.save_for_backward(q, kv, out, lse, pos, *saved)
        ctx.meta = (all_pos, group, rotator_kind, scale, save_kv)
        ctx.dbg = dbg
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, kv, out, lse, pos, *saved = ctx.saved_tensors
        all_pos, group, rotator_kind, scale, save_kv = ctx.meta
        d = ctx.dbg.d if ctx.dbg is not None else None
        skip_rot = d is not None and d.skip_dkv_rotation        # diagnostics of the reference's backward
        iter0_only = d is not None and d.iter0_only_dkv         # (ContextParallelBackward.h:102-130): wrong gradients by design
        N, r = dist.get_world_size(group), dist.get_rank(group)
        B, Tl, Hq, D = q.shape
        cuda = q.is_cuda
        # the reference forces the all-to-all rotator for gradients when the forward used all-gather
        # (ContextParallelBackward.h:204-206): gradients differ per step, there is nothing to gather once.
        grad_kind = "alltoall" if rotator_kind == "allgather" else rotator_kind
        kv_rot = make_rotator(rotator_kind, group) if not save_kv else None
        g_rot = make_rotator(grad_kind, group)
        do = do.contiguous()
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        dkv = torch.zeros(kv.shape, dtype=torch.float32, device=q.device)      # travelling accumulator
        if cuda:
            delta, lse2 = AB.flash_bwd_prep(out, do, lse)
            qpos_pad = AB.padded_q_pos(Tl, q.device, pos)
        cur = kv
        for i in range(N):
            s = (r - i) % N
            kv_handle = None
            if i < N - 1 and not save_kv:
                kv_handle = kv_rot.exchange(cur)
            for (row0, n, p0) in (_halves(all_pos[s]) if not (iter0_only and i > 0) else []):
                kb, vb = cur[0][:, row0:row0 + n], cur[1][:, row0:row0 + n]
                if cuda:
                    dkb = dkv[0][:, row0:row0 + n]
                    dvb = dkv[1][:, row0:row0 + n]
                    if not dkb.is_contiguous():
                        dkc, dvc = dkb.contiguous(), dvb.contiguous()
                        AB.flash_bwd_core(q, kb, vb, do, lse2, delta, qpos_pad, scale, True, p0, dq, dkc, dvc, True)
                        dkb.copy_(dkc); dvb.copy_(dvc)
                    else:
                        AB.flash_bwd_core(q, kb, vb, do, lse2, delta, qpos_pad, scale, True, p0, dq, dkb, dvb, True)
                else:
                    kp = torch.arange(p0, p0 + n)
                    a, b_, c = ref.attention_dense_bwd(q, kb, vb, out, lse, do, scale, pos, kp, True)
                    dq += a.float()
                    dkv[0][:, row0:row0 + n] += b_.float()
                    dkv[1][:, row0:row0 + n] += c.float()
            # pass the accumulator on: the next rank holds the same K/V block at its next step
            g_handle = g_rot.exchange(dkv) if not skip_rot else None
            if i < N - 1:
                cur = saved[i] if save_kv else kv_handle.wait()
            if g_handle is not None:
                dkv = g_handle.wait()
        dk, dv = dkv[0].to(q.dtype), dkv[1].to(q.dtype)
        return dq.to(q.dtype), dk, dv, None, None, None, None, None, None, None


def ring_attention(q, k, v, pos, all_pos, group, rotator_kind: str = "p2p", scale: Optional[float] = None,
                   save_kv: bool = False, dbg=None):
    """``all_pos[s]`` is the (CPU int64) position vector of ring rank ``s``'s shard.  ``save_kv`` keeps the N-1
    received blocks for backward (the reference's default); without it backward rotates K/V again
    (``CP_RECOMPUTE_K``, context_parallel/ContextParallelBackward.h:214-242,279-304).  ``dbg``: ``utils.debug.DebugTools``."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return _RingAttnFn.apply(q, k, v, pos, all_pos, group, rotator_kind, scale, save_kv, dbg)
