"""GPT-2 with context-parallel attention (the model of the reference's ``gpt2_cp_test`` trainer,
Scripts/Blutrain/gpt2_cp_test.cpp:201-456): learned token + position embeddings (positions are the
GLOBAL ids of the local shard, :496-513,535-538), pre-LayerNorm blocks with biased projections,
GELU(tanh) MLP of width 4·d, optional tied ``lm_head``.  Parameter names follow the PyTorch layout
used by the named-init weight files (Scripts/Pytorch/gpt2_cp_attnstyle_fp32.py:752-767).
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
from ..ops import xent
from ..parallel.cp_attention import CPAttention, CPContext


def _padded_normal(rows: int, rows_padded: int, cols: int, gen: torch.Generator) -> torch.Tensor:
    w = torch.zeros(rows_padded, cols)
    w[:rows].normal_(0.0, 0.02, generator=gen)
    return w


class GPT2Block(nn.Module):
    def __init__(self, cfg: Config, gen: torch.Generator):
        super().__init__()
        d = cfg.n_embd
        self.cfg = cfg
        resid = 0.02 / math.sqrt(2.0 * cfg.n_layer)

        def normal(shape, std):
            return nn.Parameter(torch.empty(shape).normal_(0.0, std, generator=gen))
        self.ln_1_w, self.ln_1_b = nn.Parameter(torch.ones(d)), nn.Parameter(torch.zeros(d))
        self.c_attn_w, self.c_attn_b = normal((3 * d, d), 0.02), nn.Parameter(torch.zeros(3 * d))
        self.attn_proj_w, self.attn_proj_b = normal((d, d), resid), nn.Parameter(torch.zeros(d))
        self.ln_2_w, self.ln_2_b = nn.Parameter(torch.ones(d)), nn.Parameter(torch.zeros(d))
        self.c_fc_w, self.c_fc_b = normal((4 * d, d), 0.02), nn.Parameter(torch.zeros(4 * d))
        self.mlp_proj_w, self.mlp_proj_b = normal((d, 4 * d), resid), nn.Parameter(torch.zeros(d))

    def pre_attention(self, x, pending):
        h, x = E.layernorm(x, self.ln_1_w, self.ln_1_b, 1e-5, pending)
        return x, G.linear(h, self.c_attn_w, self.c_attn_b)

    def post_attention(self, x, attn_out):
        a = G.linear(attn_out, self.attn_proj_w, self.attn_proj_b)
        h, x = E.layernorm(x, self.ln_2_w, self.ln_2_b, 1e-5, a)
        act = G.linear_gelu(h, self.c_fc_w, self.c_fc_b)
        return x, G.linear(act, self.mlp_proj_w, self.mlp_proj_b)


class GPT2(nn.Module):
    def __init__(self, cfg: Config, cp: Optional[CPContext] = None, device="cpu", seed: Optional[int] = None,
                 block_size: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        self.cp = cp or CPContext.single(cfg)
        gen = torch.Generator().manual_seed(cfg.seed if seed is None else seed)
        d = cfg.n_embd
        self.block_size = block_size or max(1024, cfg.T)
        self.wte = nn.Parameter(_padded_normal(cfg.vocab_size, cfg.vocab_padded, d, gen))
        self.wpe = nn.Parameter(torch.empty(self.block_size, d).normal_(0.0, 0.02, generator=gen))
        self.blocks = nn.ModuleList([GPT2Block(cfg, gen) for _ in range(cfg.n_layer)])
        self.ln_f_w, self.ln_f_b = nn.Parameter(torch.ones(d)), nn.Parameter(torch.zeros(d))
        self.lm_head = None if cfg.weight_tying else nn.Parameter(
            _padded_normal(cfg.vocab_size, cfg.vocab_padded, d, gen))
        self.to(device)
        self.attn = CPAttention(cfg, self.cp)

    def named_tensors(self) -> Dict[str, torch.Tensor]:
        """Parameters under the names of the named-init files: each block's first LayerNorm lives inside its
        attention module and the second inside its MLP (``transformer.h.<i>.attn.ln.*`` / ``.mlp.ln.*``,
        Scripts/Blutrain/gpt2_cp_test.cpp:909-929; Scripts/Pytorch/gpt2_cp_attnstyle_fp32.py:192,300)."""
        out: Dict[str, torch.Tensor] = {"transformer.wte.weight": self.wte, "transformer.wpe.weight": self.wpe}
        for i, b in enumerate(self.blocks):
            p = f"transformer.h.{i}."
            out[p + "attn.ln.weight"], out[p + "attn.ln.bias"] = b.ln_1_w, b.ln_1_b
            out[p + "attn.c_attn.weight"], out[p + "attn.c_attn.bias"] = b.c_attn_w, b.c_attn_b
            out[p + "attn.c_proj.weight"], out[p + "attn.c_proj.bias"] = b.attn_proj_w, b.attn_proj_b
            out[p + "mlp.ln.weight"], out[p + "mlp.ln.bias"] = b.ln_2_w, b.ln_2_b
            out[p + "mlp.c_fc.weight"], out[p + "mlp.c_fc.bias"] = b.c_fc_w, b.c_fc_b
            out[p + "mlp.c_proj.weight"], out[p + "mlp.c_proj.bias"] = b.mlp_proj_w, b.mlp_proj_b
        out["transformer.ln_f.weight"], out["transformer.ln_f.bias"] = self.ln_f_w, self.ln_f_b
        if self.lm_head is not None:
            out["lm_head.weight"] = self.lm_head
        return out

    def hidden(self, idx_local: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        x = E.embedding(idx_local, self.wte, pos, self.wpe)
        pending = None
        use_ckpt = cfg.recompute in ("selective", "full") and torch.is_grad_enabled()
        full = cfg.recompute == "full" and torch.is_grad_enabled()
        for blk in self.blocks:
            if full:
                x, pending = checkpoint(self._block, blk, x, pending, pos, use_reentrant=False)
            elif use_ckpt:
                x, qkv = checkpoint(blk.pre_attention, x, pending, use_reentrant=False)
                o = self.attn(qkv, pos)
                x, pending = checkpoint(blk.post_attention, x, o, use_reentrant=False)
            else:
                x, qkv = blk.pre_attention(x, pending)
                o = self.attn(qkv, pos)
                x, pending = blk.post_attention(x, o)
        h, _ = E.layernorm(x, self.ln_f_w, self.ln_f_b, 1e-5, pending)
        return h

    def _block(self, blk, x, pending, pos):
        """One whole block; ``CP_RECOMPUTE=full`` re-runs it (attention and its communication included) in backward."""
        x, qkv = blk.pre_attention(x, pending)
        o = self.attn(qkv, pos)
        return blk.post_attention(x, o)

    def head_weight(self) -> torch.Tensor:
        return self.wte if self.lm_head is None else self.lm_head

    def loss_sum(self, idx_local, targets_local, pos, grad_scale: float = 1.0) -> torch.Tensor:
        h = self.hidden(idx_local, pos)
        return xent.linear_cross_entropy(h, self.head_weight(), targets_local, grad_scale, self.cfg.vocab_size)

    def per_token_nll(self, idx_local, targets_local, pos) -> torch.Tensor:
        with torch.no_grad():
            h = self.hidden(idx_local, pos)
            return xent.per_token_nll(h, self.head_weight(), targets_local, self.cfg.vocab_size).view(idx_local.shape)
