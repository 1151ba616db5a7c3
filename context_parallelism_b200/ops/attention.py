"""Flash attention on tcgen05 tensor cores (``csrc/kernels/attention_fwd.cu`` / ``attention_bwd.cu``).

``flash_attention(q, k, v, ...)`` takes token-major tensors ``q [B,Tq,Hq,D]`` and ``k``/``v``
``[B,Tk,Hkv,D]`` (any 16-byte aligned strides: views into a packed QKV buffer are consumed in place),
supports GQA natively, and masks causally on GLOBAL positions: query row ``i`` has position
``q_pos[i]`` (default ``i``) and key row ``j`` has position ``k_off + j``.  That single rule covers local
attention, every HeadTail ring step and the fused ring over a position-ordered K/V buffer, so the
reference's Full / KHeadHalf / QTailHalf slicing (context_parallel/ContextParallel.h:730-784) is not
needed.  Returns ``(out [B,Tq,Hq,D], lse [B,Hq,Tq])``.

On CPU tensors the dense PyTorch reference runs instead (oracle path).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .. import _native as nv
from . import reference as ref


def _strides(t: torch.Tensor) -> Tuple[int, int, int]:
    """(head, token, batch) strides in elements of a ``[B,T,H,D]`` tensor with unit last stride."""
    assert t.stride(3) == 1, "head_dim must be contiguous"
    return t.stride(2), t.stride(1), t.stride(0)


def _ok_layout(t: torch.Tensor) -> bool:
    return (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all((s * t.element_size()) % 16 == 0 for s in t.stride()[:3]))


def flash_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, causal: bool = True,
              q_pos: Optional[torch.Tensor] = None, k_off: int = 0,
              ready: Optional[torch.Tensor] = None, ready_epoch: int = 0, block_rows: int = 0,
              out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
              segs: Optional[torch.Tensor] = None, n_segs: int = 0, n_copy: int = 0,
              o_scatter: Optional[tuple] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Forward only (no autograd).  ``q_pos`` is int32 ``[Tq]``.  ``ready``/``ready_epoch``/``block_rows``
    make the kernel wait, before it first touches K/V rows of block ``c``, until ``ready[c] >= ready_epoch``
    (used by the fused ring while remote blocks are still arriving).  ``segs``/``n_segs``/``n_copy`` add copy
    CTAs that pull the listed K/V segments from peers and bump ``ready``.  ``o_scatter = (peer_table, byte_off,
    rows_per_peer, head_off, heads_total)`` makes the epilogue store rows into their token owners' arenas
    (then ``out`` is not written)."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    if not _ok_layout(q):
        q = q.contiguous()
    if not _ok_layout(k):
        k = k.contiguous()
    if not _ok_layout(v) or v.stride() != k.stride():
        v = v.contiguous()
        if v.stride() != k.stride():
            k = k.contiguous()
    if out is None:
        out = (torch.empty((B, Tq, Hq, D), dtype=torch.bfloat16, device=q.device) if o_scatter is None
               else torch.empty((1,), dtype=torch.bfloat16, device=q.device))
    if lse is None:
        lse = torch.empty((B, Hq, Tq), dtype=torch.float32, device=q.device)
    if q_pos is not None:
        assert q_pos.dtype == torch.int32 and q_pos.numel() == Tq
    st = nv.status_for(q.device)
    qs, ks = _strides(q), _strides(k)
    nv.call("flash_fwd", nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(out), nv.ptr(lse),
            nv.i(B), nv.i(Tq), nv.i(Tk), nv.i(Hq), nv.i(Hkv), nv.i(D),
            nv.l(qs[0]), nv.l(qs[1]), nv.l(qs[2]), nv.l(ks[0]), nv.l(ks[1]), nv.l(ks[2]),
            nv.f(scale), nv.i(causal), nv.i(k_off), nv.ptr(q_pos), nv.ptr(ready), nv.i(ready_epoch),
            nv.i(block_rows), nv.ptr(segs), nv.i(n_segs), nv.i(n_copy),
            nv.ptr(o_scatter[0] if o_scatter else None), nv.l(o_scatter[1] if o_scatter else 0),
            nv.i(o_scatter[2] if o_scatter else 0), nv.i(o_scatter[3] if o_scatter else 0),
            nv.i(o_scatter[4] if o_scatter else 0), st.ptr(), nv.stream_ptr(q.device))
    return out, lse


def flash_bwd(q, k, v, o, lse, do, scale: float, causal: bool = True, q_pos=None, k_off: int = 0,
              dq: Optional[torch.Tensor] = None, dk: Optional[torch.Tensor] = None,
              dv: Optional[torch.Tensor] = None, dkv_accumulate: bool = False):
    """Backward from the merged LSE.  Returns ``(dq, dk, dv)`` as bf16 tensors shaped like q/k/v unless fp32
    accumulation buffers ``dk``/``dv`` ``[B,Tk,Hkv,D]`` are supplied (ring: contributions of several
    calls are summed in fp32, the reference's travelling accumulator is fp32 too,
    context_parallel/ContextParallelBackward.h:151-158)."""
    from .attention_bwd import flash_bwd_cuda
    return flash_bwd_cuda(q, k, v, o, lse, do, scale, causal, q_pos, k_off, dq, dk, dv, dkv_accumulate)


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, q_pos, k_off):
        out, lse = flash_fwd(q, k, v, scale, causal, q_pos, k_off)
        ctx.save_for_backward(q, k, v, out, lse, q_pos)
        ctx.scale, ctx.causal, ctx.k_off = scale, causal, k_off
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, out, lse, q_pos = ctx.saved_tensors
        dq, dk, dv = flash_bwd(q, k, v, out, lse, dout, ctx.scale, ctx.causal, q_pos, ctx.k_off)
        return dq, dk, dv, None, None, None, None


# ATTN_FP32=1: differentiable attention goes through the fp32-accurate CUDA-core kernels (parity runs); set by the engine.
FP32_ACCURATE = False


def _fp32_args(q, k, B, Tq, Tk, Hq, Hkv, D, scale, causal, k_off, q_pos):
    qs, ks = _strides(q), _strides(k)
    return (nv.i(B), nv.i(Tq), nv.i(Tk), nv.i(Hq), nv.i(Hkv), nv.i(D), nv.l(qs[0]), nv.l(qs[1]), nv.l(qs[2]), nv.l(ks[0]), nv.l(ks[1]),
            nv.l(ks[2]), nv.f(scale), nv.i(causal), nv.i(k_off), nv.ptr(q_pos), nv.stream_ptr(q.device))


class _AttnFp32Fn(torch.autograd.Function):
    """The fp32-accurate variant (``csrc/kernels/attention_fp32.cu``; the reference's ``ATTN_FP32`` scalar kernel,
    context_parallel/FusedSDPAOp.h:134-163): bf16 inputs, every intermediate in fp32, fp32 gradients rounded once."""

    @staticmethod
    def forward(ctx, q, k, v, scale, causal, q_pos, k_off):
        B, Tq, Hq, D = q.shape
        Tk, Hkv = k.shape[1], k.shape[2]
        q = q if _ok_layout(q) else q.contiguous()
        k = k if _ok_layout(k) else k.contiguous()
        if not _ok_layout(v) or v.stride() != k.stride():
            k, v = k.contiguous(), v.contiguous()
        qp = None if q_pos is None else q_pos.to(torch.int32)
        out = torch.empty((B, Tq, Hq, D), dtype=torch.float32, device=q.device)
        lse = torch.empty((B, Hq, Tq), dtype=torch.float32, device=q.device)
        nv.call("attn_fp32_fwd", nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(out), nv.ptr(lse),
                *_fp32_args(q, k, B, Tq, Tk, Hq, Hkv, D, scale, causal, k_off, qp))
        ctx.save_for_backward(q, k, v, out, lse, qp)
        ctx.scale, ctx.causal, ctx.k_off = scale, causal, k_off
        ctx.mark_non_differentiable(lse)
        return out.to(q.dtype), lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, out, lse, qp = ctx.saved_tensors
        B, Tq, Hq, D = q.shape
        Tk, Hkv = k.shape[1], k.shape[2]
        do = dout.float().contiguous()
        dq = torch.empty((B, Tq, Hq, D), dtype=torch.float32, device=q.device)
        dk = torch.zeros((B, Tk, Hkv, D), dtype=torch.float32, device=q.device)
        dv = torch.zeros_like(dk)
        nv.call("attn_fp32_bwd", nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(out), nv.ptr(lse), nv.ptr(do), nv.ptr(dq), nv.ptr(dk), nv.ptr(dv),
                *_fp32_args(q, k, B, Tq, Tk, Hq, Hkv, D, ctx.scale, ctx.causal, ctx.k_off, qp))
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None, None


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
                    causal: bool = True, q_pos: Optional[torch.Tensor] = None, k_off: int = 0
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Differentiable attention; see the module docstring for layouts and masking."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if q.is_cuda and FP32_ACCURATE:
        return _AttnFp32Fn.apply(q, k, v, scale, causal, q_pos, k_off)
    if q.is_cuda:
        return _FlashAttnFn.apply(q, k, v, scale, causal, q_pos, k_off)
    Tk = k.shape[1]
    kp = torch.arange(k_off, k_off + Tk)
    return ref.attention_dense(q, k, v, scale, q_pos, kp, causal)
