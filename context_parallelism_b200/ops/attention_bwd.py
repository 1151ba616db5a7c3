"""Host wrapper of the tcgen05 flash-attention backward (``csrc/kernels/attention_bwd.cu``)."""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _native as nv
from .attention import _ok_layout, _strides

_INT_MAX = 2 ** 31 - 1
# CPB_BWD_GENERAL=1 routes head_dim 64 through the general kernel as well (comparison / fallback)
_USE_GENERAL_D64 = os.environ.get("CPB_BWD_GENERAL", "0") == "1"


def padded_q_pos(Tq: int, device, q_pos: Optional[torch.Tensor]) -> torch.Tensor:
    tq_pad = (Tq + 127) // 128 * 128
    out = torch.full((tq_pad,), _INT_MAX, dtype=torch.int32, device=device)
    if q_pos is None:
        out[:Tq] = torch.arange(Tq, dtype=torch.int32, device=device)
    else:
        out[:Tq] = q_pos.to(torch.int32)
    return out


def flash_bwd_prep(o: torch.Tensor, do: torch.Tensor, lse: torch.Tensor):
    """``delta = rowsum(dO∘O)`` and ``lse·log2(e)`` padded to a multiple of 128 rows."""
    B, Tq, Hq, D = o.shape
    tq_pad = (Tq + 127) // 128 * 128
    delta = torch.empty((B, Hq, tq_pad), dtype=torch.float32, device=o.device)
    lse2 = torch.empty_like(delta)
    nv.call("flash_bwd_prep", nv.ptr(o), nv.ptr(do), nv.ptr(lse), nv.ptr(delta), nv.ptr(lse2),
            nv.i(B), nv.i(Tq), nv.i(Hq), nv.i(D), nv.i(tq_pad), nv.stream_ptr(o.device))
    return delta, lse2


def flash_bwd_delta(o: torch.Tensor, do: torch.Tensor) -> torch.Tensor:
    """Only ``delta = rowsum(dO∘O)`` ``[B,Hq,Tq_pad]`` (computed where the tokens live)."""
    B, Tq, Hq, D = o.shape
    tq_pad = (Tq + 127) // 128 * 128
    delta = torch.empty((B, Hq, tq_pad), dtype=torch.float32, device=o.device)
    nv.call("flash_bwd_prep", nv.ptr(o), nv.ptr(do), nv.ptr(None), nv.ptr(delta), nv.ptr(None),
            nv.i(B), nv.i(Tq), nv.i(Hq), nv.i(D), nv.i(tq_pad), nv.stream_ptr(o.device))
    return delta


def flash_bwd_lse2(lse: torch.Tensor, D: int) -> torch.Tensor:
    """Only ``lse·log2(e)`` padded ``[B,Hq,Tq_pad]``."""
    B, Hq, Tq = lse.shape
    tq_pad = (Tq + 127) // 128 * 128
    lse2 = torch.empty((B, Hq, tq_pad), dtype=torch.float32, device=lse.device)
    nv.call("flash_bwd_prep", nv.ptr(None), nv.ptr(None), nv.ptr(lse), nv.ptr(None), nv.ptr(lse2),
            nv.i(B), nv.i(Tq), nv.i(Hq), nv.i(D), nv.i(tq_pad), nv.stream_ptr(lse.device))
    return lse2


def flash_bwd_core(q, k, v, do, lse2, delta, qpos_pad, scale, causal, k_off, dq_f32, dk, dv, dkv_accumulate,
                   route=None):
    """One launch of the backward kernel: ``dq_f32`` (fp32) is accumulated with atomics; ``dk``/``dv`` are
    written as bf16, or accumulated in fp32 when ``dkv_accumulate``.  ``route = (route_k, route_v, rows, tl)``
    (int64 device tables of per-chunk owner addresses) makes the epilogue add each dK/dV tile into its owner's
    fp32 accumulator over NVLink instead."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    st = nv.status_for(q.device)
    qs, ks = _strides(q), _strides(k)
    assert v.stride() == k.stride()
    if D == 64 and not _USE_GENERAL_D64:
        # head_dim 64 kernel (csrc/kernels/attention_bwd64.cu): the per-row vectors enter the tensor-core products as
        # three-term bf16 splits, produced here from the fp32 vectors (a few tens of microseconds)
        n = lse2.numel()
        aug = torch.empty((2, n, 8), dtype=torch.bfloat16, device=q.device)
        nv.call("flash_bwd64_aug", nv.ptr(lse2), nv.ptr(delta), nv.ptr(aug[0]), nv.ptr(aug[1]), nv.l(n), nv.f(scale),
                nv.stream_ptr(q.device))
        nv.call("flash_bwd64", nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(do), nv.ptr(aug[0]), nv.ptr(aug[1]), nv.ptr(dq_f32),
                nv.ptr(dk), nv.ptr(dv), nv.i(B), nv.i(Tq), nv.i(Tk), nv.i(Hq), nv.i(Hkv), nv.i(lse2.shape[-1]),
                nv.l(qs[0]), nv.l(qs[1]), nv.l(qs[2]), nv.l(ks[0]), nv.l(ks[1]), nv.l(ks[2]),
                nv.f(scale), nv.i(causal), nv.i(k_off), nv.ptr(qpos_pad), nv.i(2 if route is not None else int(dkv_accumulate)),
                nv.ptr(route[0] if route else None), nv.ptr(route[1] if route else None),
                nv.i(route[2] if route else 0), nv.i(route[3] if route else 0), st.ptr(), nv.stream_ptr(q.device))
        return
    nv.call("flash_bwd", nv.ptr(q), nv.ptr(k), nv.ptr(v), nv.ptr(do), nv.ptr(lse2), nv.ptr(delta), nv.ptr(dq_f32),
            nv.ptr(dk), nv.ptr(dv), nv.i(B), nv.i(Tq), nv.i(Tk), nv.i(Hq), nv.i(Hkv), nv.i(D), nv.i(lse2.shape[-1]),
            nv.l(qs[0]), nv.l(qs[1]), nv.l(qs[2]), nv.l(ks[0]), nv.l(ks[1]), nv.l(ks[2]),
            nv.f(scale), nv.i(causal), nv.i(k_off), nv.ptr(qpos_pad), nv.i(2 if route is not None else int(dkv_accumulate)),
            nv.ptr(route[0] if route else None), nv.ptr(route[1] if route else None),
            nv.i(route[2] if route else 0), nv.i(route[3] if route else 0), st.ptr(), nv.stream_ptr(q.device))


def cast_to_bf16(x_f32: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    out = torch.empty(x_f32.shape, dtype=torch.bfloat16, device=x_f32.device)
    nv.call("cast_f32_bf16", nv.ptr(x_f32), nv.ptr(out), nv.l(x_f32.numel()), nv.f(scale), nv.stream_ptr(x_f32.device))
    return out


def flash_bwd_cuda(q, k, v, o, lse, do, scale, causal=True, q_pos=None, k_off=0,
                   dq=None, dk=None, dv=None, dkv_accumulate=False):
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
    do = do.contiguous()
    o = o.contiguous()
    delta, lse2 = flash_bwd_prep(o, do, lse)
    qpos_pad = padded_q_pos(Tq, q.device, q_pos)
    dq_f32 = torch.zeros((B, Tq, Hq, D), dtype=torch.float32, device=q.device) if dq is None else dq
    if dkv_accumulate:
        assert dk is not None and dv is not None and dk.dtype == torch.float32
    else:
        dk = torch.empty((B, Tk, Hkv, D), dtype=torch.bfloat16, device=q.device)
        dv = torch.empty_like(dk)
    flash_bwd_core(q, k, v, do, lse2, delta, qpos_pad, scale, causal, k_off, dq_f32, dk, dv, dkv_accumulate)
    if dq is None:
        return cast_to_bf16(dq_f32), dk, dv
    return dq_f32, dk, dv
