"""Memory-bound ops (``csrc/kernels/elementwise.cu``): norms with fused residual add, activation
backward, bias gradient, embedding, QK-norm + RoPE on packed QKV, LSE merge.

Each public function takes CUDA bf16 tensors and launches our kernel, or CPU tensors and runs the
PyTorch reference (oracle path).  Parameters that carry ``main_grad`` get their gradients
accumulated there in fp32.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native as nv
from . import reference as ref
from .gemm import accumulate_vec_grad


# ----------------------------------------------------------------------------- raw launchers
def bias_grad_into(dy2: torch.Tensor, buf: torch.Tensor) -> None:
    nv.call("bias_grad", nv.ptr(dy2), nv.ptr(buf), nv.i(dy2.shape[0]), nv.i(dy2.shape[1]), nv.stream_ptr(dy2.device))


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    Fh = gu.shape[-1] // 2
    gu2 = gu.reshape(-1, 2 * Fh)
    act = torch.empty((gu2.shape[0], Fh), dtype=gu.dtype, device=gu.device)
    nv.call("swiglu_fwd", nv.ptr(gu2), nv.ptr(act), nv.l(gu2.shape[0]), nv.i(Fh), nv.stream_ptr(gu.device))
    return act.view(*gu.shape[:-1], Fh)


def swiglu_bwd(gu: torch.Tensor, dact: torch.Tensor) -> torch.Tensor:
    Fh = gu.shape[-1] // 2
    dgu = torch.empty_like(gu)
    nv.call("swiglu_bwd", nv.ptr(gu), nv.ptr(dact), nv.ptr(dgu), nv.l(gu.numel() // (2 * Fh)), nv.i(Fh),
            nv.stream_ptr(gu.device))
    return dgu


def gelu_fwd(x: torch.Tensor) -> torch.Tensor:
    y = torch.empty_like(x)
    nv.call("gelu", nv.ptr(x), nv.ptr(None), nv.ptr(y), nv.l(x.numel()), nv.i(0), nv.stream_ptr(x.device))
    return y


def gelu_bwd(pre: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    dx = torch.empty_like(pre)
    nv.call("gelu", nv.ptr(pre), nv.ptr(dy), nv.ptr(dx), nv.l(pre.numel()), nv.i(1), nv.stream_ptr(pre.device))
    return dx


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if not a.is_cuda:
        return a + b
    a, b = a.contiguous(), b.contiguous()
    y = torch.empty_like(a)
    nv.call("add_bf16", nv.ptr(a), nv.ptr(b), nv.ptr(y), nv.l(a.numel()), nv.stream_ptr(a.device))
    return y


# ----------------------------------------------------------------------------- norms
class _NormFn(torch.autograd.Function):
    """``y = norm(x [+ res])``; returns ``(y, x_new)`` where ``x_new = x + res`` (or ``x``)."""
    @staticmethod
    def forward(ctx, x, res, w, b, eps, layer):
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        stats = torch.empty((rows, 2), dtype=torch.float32, device=x.device)
        if res is not None:
            r2 = res.reshape(-1, d)
            if not r2.is_contiguous():
                r2 = r2.contiguous()
            xnew = torch.empty_like(x2)
        else:
            r2, xnew = None, x2
        nv.call("norm_fwd", nv.ptr(x2), nv.ptr(r2), nv.ptr(w), nv.ptr(b), nv.ptr(xnew), nv.ptr(y), nv.ptr(stats),
                nv.i(rows), nv.i(d), nv.f(eps), nv.i(layer), nv.stream_ptr(x.device))
        ctx.save_for_backward(xnew, stats)
        ctx.w, ctx.b, ctx.layer, ctx.has_res = w, b, layer, res is not None
        ctx.shape = x.shape
        ctx.set_materialize_grads(False)
        return y.view(x.shape), xnew.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dxnew):
        xnew, stats = ctx.saved_tensors
        w = ctx.w
        d = xnew.shape[-1]
        if dy is None:
            dy = torch.zeros(ctx.shape, dtype=xnew.dtype, device=xnew.device)
        dy2 = dy.reshape(-1, d)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres2 = None
        if dxnew is not None:
            dres2 = dxnew.reshape(-1, d)
            if not dres2.is_contiguous():
                dres2 = dres2.contiguous()
        dx = torch.empty_like(xnew)
        wp, bp = ctx.w, ctx.b
        dw_buf = getattr(wp, "main_grad", None) if wp is not None else None
        db_buf = getattr(bp, "main_grad", None) if bp is not None else None
        own_dw = own_db = None
        if wp is not None and dw_buf is None:
            own_dw = dw_buf = torch.zeros(d, dtype=torch.float32, device=dy.device)
        if bp is not None and db_buf is None:
            own_db = db_buf = torch.zeros(d, dtype=torch.float32, device=dy.device)
        nv.call("norm_bwd", nv.ptr(xnew), nv.ptr(dy2), nv.ptr(dres2), nv.ptr(w), nv.ptr(stats), nv.ptr(dx),
                nv.ptr(dw_buf), nv.ptr(db_buf), nv.i(xnew.shape[0]), nv.i(d), nv.i(ctx.layer), nv.stream_ptr(dy.device))
        for prm in (wp, bp):
            hook = getattr(prm, "_grad_ready", None) if prm is not None else None
            if hook is not None:
                hook(prm)
        dx = dx.view(ctx.shape)
        return (dx, dx if ctx.has_res else None,
                None if own_dw is None else own_dw.to(wp.dtype), None if own_db is None else own_db.to(bp.dtype),
                None, None)


def rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, residual: Optional[torch.Tensor] = None
            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(rmsnorm(x + residual) * w, x + residual)``."""
    if x.is_cuda:
        return _NormFn.apply(x, residual, w, None, eps, 0)
    xn = x if residual is None else x + residual
    return ref.rmsnorm(xn, w, eps), xn


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float,
              residual: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    if x.is_cuda:
        return _NormFn.apply(x, residual, w, b, eps, 1)
    xn = x if residual is None else x + residual
    return ref.layernorm(xn, w, b, eps), xn


# ----------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, pos, wte, wpe):
        idx2 = idx.reshape(-1).contiguous().long()
        d = wte.shape[1]
        out = torch.empty((idx2.numel(), d), dtype=wte.dtype, device=wte.device)
        period = pos.numel() if pos is not None else 1
        nv.call("embedding_fwd", nv.ptr(idx2), nv.ptr(pos), nv.ptr(wte), nv.ptr(wpe), nv.ptr(out),
                nv.l(idx2.numel()), nv.i(d), nv.i(period), nv.stream_ptr(wte.device))
        ctx.save_for_backward(idx2, pos)
        ctx.wte, ctx.wpe, ctx.period = wte, wpe, period
        return out.view(*idx.shape, d)

    @staticmethod
    def backward(ctx, dout):
        idx2, pos = ctx.saved_tensors
        wte, wpe = ctx.wte, ctx.wpe
        d = wte.shape[1]
        d2 = dout.reshape(-1, d)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        own = {}

        def buf_for(p):
            mg = getattr(p, "main_grad", None)
            if mg is None:
                mg = own[id(p)] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
            return mg
        gte = buf_for(wte)
        gpe = buf_for(wpe) if wpe is not None else None
        nv.call("embedding_bwd", nv.ptr(idx2), nv.ptr(pos), nv.ptr(d2), nv.ptr(gte), nv.ptr(gpe),
                nv.l(idx2.numel()), nv.i(d), nv.i(ctx.period), nv.stream_ptr(d2.device))
        for prm in (wte, wpe):
            hook = getattr(prm, "_grad_ready", None) if prm is not None else None
            if hook is not None:
                hook(prm)
        return (None, None, own[id(wte)].to(wte.dtype) if id(wte) in own else None,
                (own[id(wpe)].to(wpe.dtype) if wpe is not None and id(wpe) in own else None))


def embedding(idx: torch.Tensor, wte: torch.Tensor, pos: Optional[torch.Tensor] = None,
              wpe: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``wte[idx] (+ wpe[pos])``; ``idx`` is ``[B, T]``, ``pos`` is ``[T]`` global positions (the learned
    position table must be indexed with GLOBAL positions of the local shard,
    Scripts/Blutrain/gpt2_cp_test.cpp:496-513,535-538)."""
    if wte.is_cuda:
        return _EmbeddingFn.apply(idx, pos, wte, wpe)
    out = wte[idx]
    if wpe is not None:
        out = out + wpe[pos][None]
    return out


# ----------------------------------------------------------------------------- QK-norm + RoPE
class _QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, gq, gk, cache, pos, Hq, Hkv, D, eps):
        B, T = qkv.shape[0], qkv.shape[1]
        qkv_c = qkv if qkv.is_contiguous() else qkv.contiguous()
        out = torch.empty_like(qkv_c)
        st = nv.status_for(qkv.device)
        nv.call("qk_norm_rope_fwd", nv.ptr(qkv_c), nv.ptr(out), nv.ptr(gq), nv.ptr(gk), nv.ptr(cache), nv.ptr(pos),
                nv.ptr(None), nv.l(B * T), nv.i(T), nv.i(Hq), nv.i(Hkv), nv.i(D), nv.f(eps),
                nv.i(cache.shape[0] if cache is not None else 0), st.ptr(), nv.stream_ptr(qkv.device))
        ctx.save_for_backward(qkv_c, cache, pos)
        ctx.gq, ctx.gk, ctx.dims, ctx.eps = gq, gk, (B, T, Hq, Hkv, D), eps
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, cache, pos = ctx.saved_tensors
        B, T, Hq, Hkv, D = ctx.dims
        dout = dout if dout.is_contiguous() else dout.contiguous()
        din = torch.empty_like(qkv)
        gq, gk = ctx.gq, ctx.gk
        own = {}

        def buf_for(p):
            if p is None:
                return None
            mg = getattr(p, "main_grad", None)
            if mg is None:
                mg = own[id(p)] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
            return mg
        bq, bk = buf_for(gq), buf_for(gk)
        nv.call("qk_norm_rope_bwd", nv.ptr(qkv), nv.ptr(dout), nv.ptr(din), nv.ptr(gq), nv.ptr(gk), nv.ptr(cache),
                nv.ptr(pos), nv.ptr(bq), nv.ptr(bk), nv.l(B * T), nv.i(T), nv.i(Hq), nv.i(Hkv), nv.i(D), nv.f(ctx.eps),
                nv.i(cache.shape[0] if cache is not None else 0), nv.stream_ptr(qkv.device))
        for prm in (gq, gk):
            hook = getattr(prm, "_grad_ready", None) if prm is not None else None
            if hook is not None:
                hook(prm)
        return (din, own[id(gq)].to(gq.dtype) if gq is not None and id(gq) in own else None,
                own[id(gk)].to(gk.dtype) if gk is not None and id(gk) in own else None,
                None, None, None, None, None, None)


def qk_norm_rope(qkv: torch.Tensor, gq: Optional[torch.Tensor], gk: Optional[torch.Tensor],
                 cache: Optional[torch.Tensor], pos: Optional[torch.Tensor], Hq: int, Hkv: int, D: int,
                 eps: float) -> torch.Tensor:
    """Packed ``[B, T, (Hq+2·Hkv)·D]``: RMS-norm(γ) then NeoX RoPE at ``pos[t]`` on every q and k head;
    v is passed through.  The reference re-applies norm+RoPE to each K tile for every Q tile inside
    its attention kernel (context_parallel/GQA_fused_fwd_sm103_cp.cu:188-189); here it is applied once."""
    if qkv.is_cuda:
        return _QKNormRopeFn.apply(qkv, gq, gk, cache, pos, Hq, Hkv, D, eps)
    B, T = qkv.shape[:2]
    x = qkv.view(B, T, Hq + 2 * Hkv, D)
    q = ref.qk_norm_rope(x[:, :, :Hq], gq, eps, cache, pos)
    k = ref.qk_norm_rope(x[:, :, Hq:Hq + Hkv], gk, eps, cache, pos)
    return torch.cat([q, k, x[:, :, Hq + Hkv:]], dim=2).reshape(B, T, -1)


# ----------------------------------------------------------------------------- LSE merge
def lse_merge_(out: torch.Tensor, lse: torch.Tensor, blk_out: torch.Tensor, blk_lse: torch.Tensor,
               t_begin: int = 0) -> None:
    """In-place online-softmax merge of a partial attention result into ``(out, lse)`` for local rows
    ``[t_begin, T)``; ``blk_out``/``blk_lse`` hold exactly those rows (``t_begin = T/2`` is the reference's
    ``partial`` second-half update, context_parallel/SDPAMerger.h:91-102)."""
    B, T, H, D = out.shape
    if out.is_cuda:
        nv.call("lse_merge", nv.ptr(out), nv.ptr(lse), nv.ptr(blk_out.contiguous()), nv.ptr(blk_lse.contiguous()),
                nv.i(B), nv.i(T), nv.i(H), nv.i(D), nv.i(t_begin), nv.i(blk_out.shape[1]), nv.i(t_begin),
                nv.stream_ptr(out.device))
        return
    o, l = ref.lse_merge(out[:, t_begin:], lse[:, :, t_begin:], blk_out, blk_lse)
    out[:, t_begin:] = o
    lse[:, :, t_begin:] = l
