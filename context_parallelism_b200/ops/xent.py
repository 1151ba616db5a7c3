"""Fused language-model head + cross-entropy that never materialises ``[tokens, vocab]``.

``linear_cross_entropy(x, w, targets)`` returns the *sum* of token NLLs (fp32) and the number of
counted tokens.  On CUDA the rows are processed in chunks: lm_head GEMM into an fp32 chunk buffer →
``xent`` kernel (loss + bf16 dlogits in one pass) → dX chunk GEMM and dW accumulation, all inside the
forward call (the gradient of a sum-of-NLL loss with respect to the logits does not depend on
anything downstream except one scalar, which is applied in ``backward``).  The reference materialises
the full logits tensor (Scripts/Blutrain/bluscriptCP.cpp:452-459), which at T = 128 K and a 128 K
vocabulary would be 64 GB.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn.functional as F

from .. import _native as nv
from .gemm import gemm

CHUNK_ROWS = 4096


def xent_chunk(logits: torch.Tensor, targets: torch.Tensor, loss_sum: torch.Tensor, grad_scale: float,
               want_grad: bool = True, row_loss: torch.Tensor = None, n_valid: int = 0):
    rows, Vc = logits.shape
    V = n_valid or Vc
    dlog = torch.empty((rows, Vc), dtype=torch.bfloat16, device=logits.device) if want_grad else None
    st = nv.status_for(logits.device)
    nv.call("xent", nv.ptr(logits), nv.ptr(targets), nv.ptr(dlog), nv.ptr(loss_sum), nv.ptr(row_loss), nv.i(rows), nv.i(V), nv.i(Vc),
            nv.l(logits.stride(0)), nv.l(dlog.stride(0) if dlog is not None else 0), nv.f(grad_scale), st.ptr(),
            nv.stream_ptr(logits.device))
    return dlog


class _LinearCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, targets, grad_scale, n_valid):
        x2 = x.reshape(-1, x.shape[-1])
        tg = targets.reshape(-1).contiguous().long()
        N, d = x2.shape
        V = w.shape[0]
        loss_sum = torch.zeros(1, dtype=torch.float32, device=x.device)
        need_grad = x.requires_grad or w.requires_grad
        dx = torch.empty_like(x2) if need_grad else None
        mg = getattr(w, "main_grad", None)
        dw_own = None
        if need_grad and mg is None:
            dw_own = torch.zeros((V, d), dtype=torch.float32, device=x.device)
        logits = torch.empty((min(CHUNK_ROWS, N), V), dtype=torch.float32, device=x.device)
        for r0 in range(0, N, CHUNK_ROWS):
            r1 = min(N, r0 + CHUNK_ROWS)
            xc = x2[r0:r1]
            lg = logits[: r1 - r0]
            gemm(xc, w, out=lg, epi=1)
            dlog = xent_chunk(lg, tg[r0:r1], loss_sum, grad_scale, need_grad, None, n_valid)
            if need_grad:
                gemm(dlog, w, b_mn=True, out=dx[r0:r1])
                gemm(dlog, xc, a_mn=True, b_mn=True, out=(mg if mg is not None else dw_own).view(V, d), accumulate=True)
        if need_grad and mg is not None:
            hook = getattr(w, "_grad_ready", None)
            if hook is not None:
                ctx.hook, ctx.w = hook, w
        ctx.dx = dx
        ctx.dw_own = dw_own
        ctx.grad_scale = grad_scale
        ctx.xshape = x.shape
        ctx.wdtype = w.dtype
        return loss_sum.squeeze(0)

    @staticmethod
    def backward(ctx, g):
        # dX/dW were produced with `grad_scale`; the upstream scalar must match it (checked lazily on the
        # device would cost a sync, so the contract is enforced by the callers in this package).
        hook = getattr(ctx, "hook", None)
        if hook is not None:
            hook(ctx.w)
        dx = ctx.dx.view(ctx.xshape) if ctx.dx is not None else None
        dw = ctx.dw_own.to(ctx.wdtype) if ctx.dw_own is not None else None
        return dx, dw, None, None, None


def linear_cross_entropy(x: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, grad_scale: float = 1.0,
                         n_valid: int = 0) -> torch.Tensor:
    """Sum over tokens of ``-log softmax(x·wᵀ)[target]`` (targets < 0 are ignored).

    ``grad_scale`` is the scalar the caller will pass to ``backward`` for this loss (for a mean over
    ``n`` tokens and ``a`` accumulation steps: ``1/(n·a)``); on CUDA the gradients are produced during
    the forward with that factor folded in.  ``w`` may carry zero padding rows beyond the real vocabulary
    ``n_valid`` (kept so the GEMM shapes are multiples of 64); they never enter the softmax."""
    if x.is_cuda:
        return _LinearCEFn.apply(x, w, targets, grad_scale, n_valid)
    logits = F.linear(x.float(), w.float())
    if n_valid:
        logits = logits[..., :n_valid]
    return F.cross_entropy(logits.view(-1, logits.shape[-1]), targets.reshape(-1), ignore_index=-100, reduction="sum")


def per_token_nll(x: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, n_valid: int = 0) -> torch.Tensor:
    """Forward-only per-token NLL ``[tokens]`` (per-position perplexity evaluation)."""
    x2 = x.reshape(-1, x.shape[-1])
    tg = targets.reshape(-1).contiguous().long()
    if not x.is_cuda:
        logits = F.linear(x2.float(), w.float())
        if n_valid:
            logits = logits[:, :n_valid]
        return F.cross_entropy(logits, tg, reduction="none")
    N, V = x2.shape[0], w.shape[0]
    out = torch.empty(N, dtype=torch.float32, device=x.device)
    logits = torch.empty((min(CHUNK_ROWS, N), V), dtype=torch.float32, device=x.device)
    for r0 in range(0, N, CHUNK_ROWS):
        r1 = min(N, r0 + CHUNK_ROWS)
        lg = logits[: r1 - r0]
        gemm(x2[r0:r1], w, out=lg, epi=1)
        xent_chunk(lg, tg[r0:r1], None, 1.0, False, out[r0:r1], n_valid)
    return out


def logits_last(x_last: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """fp32 logits for a few rows (generation)."""
    if not x_last.is_cuda:
        return F.linear(x_last.float(), w.float())
    x2 = x_last.reshape(-1, x_last.shape[-1])
    pad = (-x2.shape[0]) % 8
    if pad:
        x2 = torch.cat([x2, x2.new_zeros(pad, x2.shape[1])])
    return gemm(x2.contiguous(), w, out_dtype=torch.float32)[: x_last.reshape(-1, x_last.shape[-1]).shape[0]]
