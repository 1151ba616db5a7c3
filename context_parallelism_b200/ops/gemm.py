"""bf16 GEMM on tcgen05 tensor cores (``csrc/kernels/gemm.cu``) and the ``Linear`` autograd op.

``linear(x, w, b)`` is ``x @ w.T + b`` with ``w`` stored ``[out, in]`` (PyTorch layout, also the
on-disk layout of the named-init format).  The backward runs the data-gradient and weight-gradient
GEMMs on the same kernel using its N-major / M-major operand modes, so no transposed copy of an
activation or weight is ever made.  Weight gradients are accumulated in fp32 straight into
``weight.main_grad`` when the parameter has one (the flat gradient buffer the bucketed all-reduce
and the optimiser consume); ``weight._grad_ready`` (if set) is called once the gradient is written
so the all-reduce of a finished bucket can start while backward continues.

Replaces ``nn::Linear`` + cuBLAS of the reference trainers (Scripts/Blutrain/bluscriptCP.cpp:212-330).
On CPU tensors the same functions run plain PyTorch (oracle path).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .. import _native as nv
from . import reference as ref

EPI_BF16, EPI_F32, EPI_F32_ACC, EPI_BF16_GELU, EPI_BF16_SWIGLU = 0, 1, 2, 3, 4


def _rowmajor2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        t = t.reshape(-1, t.shape[-1])
    if t.stride(1) != 1 or (t.stride(0) % 8) or (t.data_ptr() % 16):
        t = t.contiguous()
    return t


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         accumulate: bool = False, bias: Optional[torch.Tensor] = None, epi: Optional[int] = None,
         aux: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``C[M,N] (+)= A·B``.  ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``), ``b`` is ``[N,K]``
    (or ``[K,N]`` when ``b_mn``); both bf16.  For ``epi == EPI_BF16_SWIGLU`` ``b`` is the fused
    ``[2F,K]`` weight and the result has ``F`` columns."""
    assert a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    a = _rowmajor2d(a)
    b = _rowmajor2d(b)
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"gemm: K mismatch {K} vs {Kb}"
    if epi is None:
        epi = EPI_F32_ACC if accumulate else (EPI_F32 if out_dtype == torch.float32 else EPI_BF16)
    if epi == EPI_BF16_SWIGLU:
        assert N % 2 == 0
        N //= 2
    if out is None:
        odt = torch.float32 if epi in (EPI_F32, EPI_F32_ACC) else torch.bfloat16
        out = torch.empty((M, N), dtype=odt, device=a.device)
        assert epi != EPI_F32_ACC, "accumulate needs an output buffer"
    assert out.stride(-1) == 1 and out.dim() == 2 and out.shape[0] == M and out.shape[1] == N
    st = nv.status_for(a.device)
    nv.call("gemm_bf16", nv.ptr(a), nv.ptr(b), nv.ptr(out), nv.ptr(aux),
            nv.ptr(bias.float() if bias is not None and bias.dtype != torch.float32 else bias),
            nv.i(M), nv.i(N), nv.i(K), nv.i(a.stride(0)), nv.i(b.stride(0)), nv.i(out.stride(0)),
            nv.i(aux.stride(0) if aux is not None else 0), nv.i(a_mn), nv.i(b_mn), nv.i(epi),
            st.ptr(), nv.stream_ptr(a.device))
    return out


def accumulate_weight_grad(w: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor) -> Optional[torch.Tensor]:
    """``dW += dy2ᵀ · x2``.  Into ``w.main_grad`` (fp32) when present (returns None so autograd stores
    nothing), otherwise returns the gradient in ``w``'s dtype."""
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        gemm(dy2, x2, a_mn=True, b_mn=True, out=mg.view(w.shape[0], -1), accumulate=True)
        hook = getattr(w, "_grad_ready", None)
        if hook is not None:
            hook(w)
        return None
    return gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype)


def accumulate_vec_grad(p: Optional[torch.Tensor], compute) -> Optional[torch.Tensor]:
    """Run ``compute(buf)`` which adds a vector gradient into the fp32 buffer ``buf``."""
    if p is None:
        return None
    mg = getattr(p, "main_grad", None)
    if mg is not None:
        compute(mg)
        hook = getattr(p, "_grad_ready", None)
        if hook is not None:
            hook(p)
        return None
    buf = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
    compute(buf)
    return buf.to(p.dtype)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b):
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w, bias=b)
        # The parameter objects are kept as plain attributes: under activation recomputation the tensors handed
        # back by ``saved_tensors`` are fresh objects without ``main_grad`` / ``_grad_ready``.
        ctx.save_for_backward(x2)
        ctx.weight = w
        ctx.has_bias = b is not None
        ctx.bias = b
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (x2,), w = ctx.saved_tensors, ctx.weight
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = gemm(dy2, w, b_mn=True).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw = accumulate_weight_grad(w, dy2, x2) if ctx.needs_input_grad[1] else None
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from .elementwise import bias_grad_into
            db = accumulate_vec_grad(ctx.bias, lambda buf: bias_grad_into(dy2, buf))
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.is_cuda:
        return _LinearFn.apply(x, w, b)
    return F.linear(x, w, b)


class _LinearSwiGLUFn(torch.autograd.Function):
    """``silu(x·Wgᵀ) ∘ (x·Wuᵀ)`` with ``W = [Wg; Wu]`` fused ``[2F, d]``; the activation is applied in
    the GEMM epilogue (the reference runs a GEMM then a separate ``swiglu`` kernel,
    bluscriptCP.cpp:327-329).  The pre-activation ``[g|u]`` is saved for the backward."""
    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        Fh = w.shape[0] // 2
        gu = torch.empty((x2.shape[0], 2 * Fh), dtype=torch.bfloat16, device=x.device)
        act = gemm(x2, w, epi=EPI_BF16_SWIGLU, aux=gu)
        ctx.save_for_backward(x2, gu)
        ctx.weight = w
        ctx.xshape = x.shape
        return act.view(*x.shape[:-1], Fh)

    @staticmethod
    def backward(ctx, dact):
        from .elementwise import swiglu_bwd
        (x2, gu), w = ctx.saved_tensors, ctx.weight
        d2 = dact.reshape(-1, dact.shape[-1])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dgu = swiglu_bwd(gu, d2)
        dx = gemm(dgu, w, b_mn=True).view(ctx.xshape)
        dw = accumulate_weight_grad(w, dgu, x2)
        return dx, dw


def linear_swiglu(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    if x.is_cuda:
        return _LinearSwiGLUFn.apply(x, w)
    return ref.swiglu(F.linear(x, w))


class _LinearGELUFn(torch.autograd.Function):
    """``gelu_tanh(x·Wᵀ + b)`` with the activation in the GEMM epilogue; pre-activation saved."""
    @staticmethod
    def forward(ctx, x, w, b):
        x2 = x.reshape(-1, x.shape[-1])
        pre = torch.empty((x2.shape[0], w.shape[0]), dtype=torch.bfloat16, device=x.device)
        act = gemm(x2, w, bias=b, epi=EPI_BF16_GELU, aux=pre)
        ctx.save_for_backward(x2, pre)
        ctx.weight = w
        ctx.bias = b
        ctx.xshape = x.shape
        return act.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dact):
        from .elementwise import bias_grad_into, gelu_bwd
        (x2, pre), w = ctx.saved_tensors, ctx.weight
        d2 = dact.reshape(-1, dact.shape[-1])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dpre = gelu_bwd(pre, d2)
        dx = gemm(dpre, w, b_mn=True).view(ctx.xshape)
        dw = accumulate_weight_grad(w, dpre, x2)
        db = accumulate_vec_grad(ctx.bias, lambda buf: bias_grad_into(dpre, buf)) if ctx.bias is not None else None
        return dx, dw, db


def linear_gelu(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    if x.is_cuda:
        return _LinearGELUFn.apply(x, w, b)
    return ref.gelu_tanh(F.linear(x, w, b))
