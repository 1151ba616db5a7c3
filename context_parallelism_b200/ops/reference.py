"""Plain PyTorch restatements of every numeric op, used as the CPU path and as test oracles.

These are the math definitions the sm_100a kernels are checked against.  They run on any
device and in any float dtype (tests use fp32 / fp64 on CPU).  Sources for the math:
dense softmax attention with a global causal mask (context_parallel/SDPAOp.h:24-214),
online-softmax merge (context_parallel/SDPAMerger.h:108-121), QK-RMS-norm followed by NeoX
half-split RoPE (context_parallel/GQA_fused_fwd_sm103_cp.cu:65-115), YaRN / LongRoPE caches
(context_parallel/YARNOps.cpp:49-138,150-208).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- norms / activations
def rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if w is not None:
        y = y * w.float()
    return y.to(x.dtype)


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(), eps).to(x.dtype)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """GELU, tanh approximation (the PyTorch parity trainer uses ``approximate="tanh"``,
    Scripts/Pytorch/gpt2_cp_attnstyle_fp32.py:302)."""
    return F.gelu(x.float(), approximate="tanh").to(x.dtype)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` with the fused projection laid out ``[gate | up]`` on the last axis."""
    g, u = gu.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gu.dtype)


# ----------------------------------------------------------------------------- RoPE caches
def yarn_inv_freq(head_dim: int, base: float, scale: float = 1.0, orig_maxpos: float = 1024.0,
                  beta_fast: float = 32.0, beta_slow: float = 1.0) -> Tuple[torch.Tensor, int, int]:
    """Per-dimension inverse frequencies with the NTK-by-parts ramp (YARNOps.cpp:76-118).
    ``high`` is clamped to ``head_dim/2-1`` as the reference does on purpose."""
    half = head_dim // 2

    def find_dim(num_rot):
        return head_dim * math.log(orig_maxpos / (num_rot * 2.0 * math.pi)) / (2.0 * math.log(base))
    low = max(int(math.floor(find_dim(beta_fast))), 0)
    high = min(int(math.ceil(find_dim(beta_slow))), half - 1)
    if scale > 1.0 and low > high:
        raise ValueError(f"YaRN: bad correction range low={low} high={high}")
    denom = float(high - low)
    if denom <= 0:
        denom = 1e-3
    i = torch.arange(half, dtype=torch.float32)
    base_freq = 1.0 / torch.pow(torch.tensor(float(base), dtype=torch.float32), 2.0 * i / head_dim)
    ramp = ((i - low) / denom).clamp(0.0, 1.0)
    inv = (base_freq / scale) * ramp + base_freq * (1.0 - ramp)
    return inv, low, high


def yarn_mscale(scale: float, no_mscale: bool = False) -> float:
    return 0.1 * math.log(scale) + 1.0 if (scale > 1.0 and not no_mscale) else 1.0


def build_rope_cache(seq_len: int, head_dim: int, base: float, scale: float = 1.0,
                     orig_maxpos: float = 1024.0, beta_fast: float = 32.0, beta_slow: float = 1.0,
                     no_mscale: bool = False, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[seq_len, head_dim]`` fp32 table, row ``p`` = ``[cos(p·f_i)·m | sin(p·f_i)·m]``
    (NeoX half-split).  ``scale == 1`` is plain RoPE."""
    if head_dim % 2:
        raise ValueError("head_dim must be even")
    inv, _, _ = yarn_inv_freq(head_dim, base, scale, orig_maxpos, beta_fast, beta_slow)
    m = yarn_mscale(scale, no_mscale)
    pos = torch.arange(seq_len, dtype=torch.float32) if positions is None else positions.float()
    ang = pos[:, None] * inv[None, :]
    return torch.cat([ang.cos() * m, ang.sin() * m], dim=1).contiguous()


def validate_longrope(lam: Sequence[float], head_dim: int, n_hat: int) -> None:
    half = head_dim // 2
    if len(lam) != half:
        raise ValueError(f"longrope: lambda size ({len(lam)}) must equal head_dim/2 ({half})")
    for i, v in enumerate(lam):
        if not v >= 1.0:
            raise ValueError(f"longrope: lambda[{i}] must be >= 1")
        if i and v < lam[i - 1]:
            raise ValueError(f"longrope: lambda must be non-decreasing (violated at i={i})")
    if n_hat < 0:
        raise ValueError("longrope: n_hat must be >= 0")


def build_rope_cache_longrope(seq_len: int, head_dim: int, base: float, lam: Sequence[float],
                              n_hat: int, mscale: float = 1.0) -> torch.Tensor:
    """``angle(p,i) = p·base_freq_i / (p < n_hat ? 1 : λ_i)`` (YARNOps.cpp:189-198)."""
    validate_longrope(lam, head_dim, n_hat)
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    base_freq = 1.0 / torch.pow(torch.tensor(float(base), dtype=torch.float32), 2.0 * i / head_dim)
    pos = torch.arange(seq_len, dtype=torch.float32)
    lam_t = torch.tensor(list(lam), dtype=torch.float32)
    div = torch.where(pos[:, None] < n_hat, torch.ones(1), lam_t[None, :])
    ang = pos[:, None] * base_freq[None, :] / div
    return torch.cat([ang.cos() * mscale, ang.sin() * mscale], dim=1).contiguous()


# ----------------------------------------------------------------------------- QK-norm + RoPE
def rope_apply(x: torch.Tensor, cache: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """NeoX rotation of ``x[..., T, D]`` with rows ``cache[pos]``; fp32 math."""
    D = x.shape[-1]
    half = D // 2
    cs = cache.to(x.device)[pos.to(x.device)]
    c, s = cs[..., :half].float(), cs[..., half:].float()
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1).to(x.dtype)


def qk_norm_rope(x: torch.Tensor, gamma: Optional[torch.Tensor], eps: float,
                 cache: Optional[torch.Tensor], pos: Optional[torch.Tensor]) -> torch.Tensor:
    """RMS-norm over head_dim with gain ``gamma`` then RoPE.  ``x`` is ``[B, T, H, D]``
    (token-major) and ``pos`` is ``[T]``; either stage is skipped when its argument is None."""
    y = x
    if gamma is not None:
        y = rmsnorm(y, gamma, eps)
    if cache is not None:
        y = rope_apply(y.transpose(1, 2), cache, pos).transpose(1, 2)
    return y


# ----------------------------------------------------------------------------- attention
def attention_dense(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                    q_pos: Optional[torch.Tensor] = None, k_pos: Optional[torch.Tensor] = None,
                    causal: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense softmax attention with a mask on *global* positions.

    ``q`` is ``[B, Tq, Hq, D]``, ``k``/``v`` are ``[B, Tk, Hkv, D]`` (token-major, GQA by head
    grouping ``hq // (Hq/Hkv)``).  Returns ``(out [B,Tq,Hq,D], lse [B,Hq,Tq])`` with natural-log
    LSE; a row with no visible key gets ``out = 0`` and ``lse = -inf``."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)                       # B Hq Tq D
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        qp = torch.arange(Tq, device=q.device) if q_pos is None else q_pos.to(q.device)
        kp = torch.arange(Tk, device=q.device) if k_pos is None else k_pos.to(q.device)
        s = s.masked_fill(kp[None, :] > qp[:, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3).to(q.dtype).contiguous(), lse


def attention_dense_bwd(q, k, v, o, lse, do, scale, q_pos=None, k_pos=None, causal=True):
    """Flash-style backward from the *merged* LSE: ``P = exp(S−LSE)``, ``D = rowsum(dO∘O)``,
    ``dS = P∘(dP − D)`` (context_parallel/SDPAOp.h ``sdpa_backward_op_manual``)."""
    B, Tq, Hq, Dh = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    dof = do.float().permute(0, 2, 1, 3)
    of = o.float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        qp = torch.arange(Tq, device=q.device) if q_pos is None else q_pos.to(q.device)
        kp = torch.arange(Tk, device=q.device) if k_pos is None else k_pos.to(q.device)
        s = s.masked_fill(kp[None, :] > qp[:, None], float("-inf"))
    lse_safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - lse_safe[..., None])
    p = torch.where(torch.isinf(lse)[..., None], torch.zeros_like(p), p)
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    dsum = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - dsum) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    dk = dk.view(B, Hkv, g, Tk, Dh).sum(2)
    dv = dv.view(B, Hkv, g, Tk, Dh).sum(2)
    return (dq.permute(0, 2, 1, 3).to(q.dtype).contiguous(),
            dk.permute(0, 2, 1, 3).to(k.dtype).contiguous(),
            dv.permute(0, 2, 1, 3).to(v.dtype).contiguous())


def lse_merge(out: torch.Tensor, lse: torch.Tensor, blk_out: torch.Tensor, blk_lse: torch.Tensor
              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Online-softmax merge of two partial attentions over disjoint key sets.

    ``out`` is ``[B,T,H,D]`` and ``lse`` is ``[B,H,T]``.  Uses the numerically safe form
    ``out −= sigmoid(blk_lse−lse)·(out−blk_out)``, ``lse −= logsigmoid(lse−blk_lse)``
    (context_parallel/SDPAMerger.h:108-121); ``-inf`` partners are the identity."""
    of, bf = out.float(), blk_out.float()
    d = (blk_lse - lse)
    both_inf = torch.isinf(lse) & torch.isinf(blk_lse) & (lse < 0) & (blk_lse < 0)
    d = torch.where(both_inf, torch.zeros_like(d), d)
    w = torch.sigmoid(d).permute(0, 2, 1)[..., None]         # B T H 1
    new_out = of - w * (of - bf)
    new_lse = torch.where(both_inf, lse, lse - F.logsigmoid(-d))
    return new_out.to(out.dtype), new_lse


# ----------------------------------------------------------------------------- loss / optimiser
def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1),
                           ignore_index=ignore_index)


def linear_cross_entropy(x: torch.Tensor, w: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean token NLL of ``softmax(x @ w.T)``; ``x`` is ``[N, d]``, ``w`` is ``[V, d]``."""
    return cross_entropy(x.float() @ w.float().t(), targets)


def adamw_step(p, g, m, v, step: int, lr: float, b1: float, b2: float, eps: float, wd: float) -> None:
    """PyTorch-semantics AdamW on fp32 tensors, in place (decoupled decay, bias-corrected)."""
    p.mul_(1.0 - lr * wd)
    m.mul_(b1).add_(g, alpha=1.0 - b1)
    v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
    bc1 = 1.0 - b1 ** step
    bc2 = 1.0 - b2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
