"""Llama-style decoder with context-parallel attention.

Block: RMSNorm → fused QKV projection (GQA) → QK-RMS-norm(γ) + RoPE at global positions → context
parallel causal attention → output projection → +residual; RMSNorm → fused gate_up projection with
SwiGLU epilogue → down projection → +residual (Scripts/Blutrain/bluscriptCP.cpp:212-330).  The
sequence is sharded before the embedding, so everything outside attention runs on the local
``T/cp`` tokens (bluscriptCP.cpp:430-459).  No learned position table; untied ``lm_head`` by default.

Differences from the reference that are deliberate: the three projections wQ/wK/wV are one GEMM
(stored fused, exposed under the reference's names for checkpoints); QK-norm + RoPE are applied once
per token instead of once per (Q tile, K tile) pair inside the attention kernel; residual adds are
fused into the following norm; the loss head never materialises the logits.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from ..config import Config
from ..ops import elementwise as E
from ..ops import gemm as G
from ..ops import rope as R
from ..ops import xent
from ..parallel.cp_attention import CPAttention, CPContext


def _padded_normal(rows: int, rows_padded: int, cols: int, gen: torch.Generator) -> torch.Tensor:
    w = torch.zeros(rows_padded, cols, device=gen.device)
    w[:rows].normal_(0.0, 0.02, generator=gen)
    return w


class LlamaBlock(nn.Module):
    def __init__(self, cfg: Config, layer_idx: int, gen: torch.Generator):
        super().__init__()
        d, hq, hkv, hd, ffn = cfg.n_embd, cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.ffn_hidden
        self.cfg, self.layer_idx = cfg, layer_idx
        resid = 1.0 / math.sqrt(2.0 * cfg.n_layer)

        def normal(shape, std):
            return nn.Parameter(torch.empty(shape, device=gen.device).normal_(0.0, std, generator=gen))
        self.q_gamma = nn.Parameter(torch.ones(hd))
        self.k_gamma = nn.Parameter(torch.ones(hd))
        self.attn_norm = nn.Parameter(torch.ones(d))
        self.wqkv = normal(((hq + 2 * hkv) * hd, d), 0.02)          # rows: [wQ | wK | wV]
        self.wo = normal((d, hq * hd), 0.02 * resid)
        self.mlp_norm = nn.Parameter(torch.ones(d))
        self.gate_up = normal((2 * ffn, d), 0.02)                   # rows: [gate | up]
        self.down = normal((d, ffn), 0.02 * resid)

    # The two halves are separate functions so activation recomputation can wrap each of them while the
    # attention core (by far the most expensive part) is never recomputed.
    def pre_attention(self, x, pending, cache, pos):
        cfg = self.cfg
        h, x = E.rmsnorm(x, self.attn_norm, cfg.rms_eps, pending)
        qkv = G.linear(h, self.wqkv)
        qkv = E.qk_norm_rope(qkv, self.q_gamma, self.k_gamma, cache, pos, cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.qk_eps)
        return x, qkv

    def post_attention(self, x, attn_out):
        cfg = self.cfg
        a = G.linear(attn_out, self.wo)
        h, x = E.rmsnorm(x, self.mlp_norm, cfg.rms_eps, a)
        act = G.linear_swiglu(h, self.gate_up)
        return x, G.linear(act, self.down)


class Llama(nn.Module):
    def __init__(self, cfg: Config, cp: Optional[CPContext] = None, device="cpu", seed: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        self.cp = cp or CPContext.single(cfg)
        # Every tensor is drawn from the CPU generator (same values on every rank and on the CPU oracle) and moved to
        # the device at once, so the host never holds more than one layer of an 8B-parameter model.  CP_INIT_DEVICE=1
        # draws on the device instead (seconds instead of minutes for billions of parameters; the values then differ
        # from the CPU stream, rank 0's are broadcast to every rank either way).
        import os
        on_dev = os.environ.get("CP_INIT_DEVICE", "0") == "1" and torch.device(device).type == "cuda"
        gen = torch.Generator(device=device if on_dev else "cpu").manual_seed(cfg.seed if seed is None else seed)
        self.wte = nn.Parameter(_padded_normal(cfg.vocab_size, cfg.vocab_padded, cfg.n_embd, gen).to(device))
        self.blocks = nn.ModuleList([LlamaBlock(cfg, i, gen).to(device) for i in range(cfg.n_layer)])
        self.norm_f = nn.Parameter(torch.ones(cfg.n_embd))
        self.lm_head = None if cfg.weight_tying else nn.Parameter(
            _padded_normal(cfg.vocab_size, cfg.vocab_padded, cfg.n_embd, gen).to(device))
        self.to(device)
        self.attn = CPAttention(cfg, self.cp)
        self.rope_cache = R.build_rope_cache(cfg.T, cfg.head_dim, cfg.rope_theta, device, cfg.yarn)
        self.rope_pos_override: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ RoPE cache control
    def set_rope_cache(self, cache: torch.Tensor) -> None:
        """Swap the cos/sin table on every layer (LongRoPE / CREAM installs, ContextParallel.h:297-388)."""
        self.rope_cache = cache

    # ------------------------------------------------------------------ naming (checkpoint / named-init format)
    def named_tensors(self) -> Dict[str, torch.Tensor]:
        """Parameters under the reference's names and order (bluscriptCP.cpp:1269-1284): per layer
        ``q_gamma,k_gamma,attn_norm,wQ,wK,wV,wO,mlp_norm,gate_up,down`` then ``wte,norm_f,lm_head``.
        Linear weights are ``[out, in]``."""
        cfg = self.cfg
        nq, nkv = cfg.n_head * cfg.head_dim, cfg.n_kv_head * cfg.head_dim
        out: Dict[str, torch.Tensor] = {}
        for i, b in enumerate(self.blocks):
            p = f"layers.{i}."
            out[p + "q_gamma"] = b.q_gamma
            out[p + "k_gamma"] = b.k_gamma
            out[p + "attn_norm"] = b.attn_norm
            out[p + "wQ"] = b.wqkv[:nq]
            out[p + "wK"] = b.wqkv[nq:nq + nkv]
            out[p + "wV"] = b.wqkv[nq + nkv:]
            out[p + "wO"] = b.wo
            out[p + "mlp_norm"] = b.mlp_norm
            out[p + "gate_up"] = b.gate_up
            out[p + "down"] = b.down
        out["wte"] = self.wte
        out["norm_f"] = self.norm_f
        if self.lm_head is not None:
            out["lm_head"] = self.lm_head
        return out

    # ------------------------------------------------------------------ forward
    def hidden(self, idx_local: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """Final-norm hidden states ``[B, T_local, d]`` for local tokens at global positions ``pos``."""
        cfg = self.cfg
        x = E.embedding(idx_local, self.wte)
        pending = None
        rpos = pos if self.rope_pos_override is None else self.rope_pos_override
        use_ckpt = cfg.recompute in ("selective", "full") and torch.is_grad_enabled()
        full = cfg.recompute == "full" and torch.is_grad_enabled()
        for blk in self.blocks:
            if full:
                # full activation recompute: only the block's input survives the forward pass; backward re-runs the
                # whole block, context-parallel attention (and its communication) included, on every rank alike
                x, pending = checkpoint(self._block, blk, x, pending, rpos, pos, use_reentrant=False)
            elif use_ckpt:
                x, qkv = checkpoint(blk.pre_attention, x, pending, self.rope_cache, rpos, use_reentrant=False)
                o = self.attn(qkv, pos)
                x, pending = checkpoint(blk.post_attention, x, o, use_reentrant=False)
            else:
                x, qkv = blk.pre_attention(x, pending, self.rope_cache, rpos)
                o = self.attn(qkv, pos)
                x, pending = blk.post_attention(x, o)
        h, _ = E.rmsnorm(x, self.norm_f, cfg.rms_eps, pending)
        return h

    def _block(self, blk, x, pending, rpos, pos):
        x, qkv = blk.pre_attention(x, pending, self.rope_cache, rpos)
        o = self.attn(qkv, pos)
        return blk.post_attention(x, o)

    def head_weight(self) -> torch.Tensor:
        return self.wte if self.lm_head is None else self.lm_head

    def loss_sum(self, idx_local, targets_local, pos, grad_scale: float = 1.0) -> torch.Tensor:
        """Sum of token NLLs over the local shard (fp32 scalar)."""
        h = self.hidden(idx_local, pos)
        return xent.linear_cross_entropy(h, self.head_weight(), targets_local, grad_scale, self.cfg.vocab_size)

    def per_token_nll(self, idx_local, targets_local, pos) -> torch.Tensor:
        with torch.no_grad():
            h = self.hidden(idx_local, pos)
            return xent.per_token_nll(h, self.head_weight(), targets_local, self.cfg.vocab_size).view(idx_local.shape)
