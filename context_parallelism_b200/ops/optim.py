"""Flat parameter storage, fused gradient-norm clipping and AdamW.

``FlatParams`` packs every parameter of a model into a few flat buffers: fp32 master weights, fp32
gradients, fp32 Adam moments and (on CUDA) a bf16 compute copy of the matrices.  Parameters become
views; ``p.main_grad`` is the fp32 gradient view our backward kernels accumulate into directly.  One
``sumsq`` launch gives the global gradient norm on the device, and one ``adamw`` launch per
decay-group applies clip + decoupled weight decay + Adam and refreshes the bf16 copy, with no host
synchronisation (the reference does `clip_grad_norm_`, a manual decay loop over parameters and
`AdamW.step`, Scripts/Blutrain/bluscriptCP.cpp:1736-1744).  A non-finite norm skips the step and sets
a flag instead of poisoning the weights (the reference aborts on NaN loss, bluscriptCP.cpp:1730-1733).

Semantics follow ``torch.optim.AdamW`` (bias correction, eps outside the square root, decay on
parameters with ``dim >= 2`` only).
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .. import _native as nv
from . import reference as ref


class FlatParams:
    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], bf16_matrices: bool):
        seen, decay, nodecay = set(), [], []
        for name, p in named_params:
            if id(p) in seen or not p.requires_grad:
                continue
            seen.add(id(p))
            (decay if p.dim() >= 2 else nodecay).append((name, p))
        self.entries: List[Tuple[str, torch.nn.Parameter, int, int]] = []
        off = 0
        for name, p in decay + nodecay:
            n = p.numel()
            self.entries.append((name, p, off, n))
            off += (n + 63) // 64 * 64          # keep every view 256-byte aligned
        self.n_decay = sum(((p.numel() + 63) // 64 * 64) for _, p in decay)
        self.total = off
        dev = (decay + nodecay)[0][1].device
        self.device = dev
        self.bf16 = bool(bf16_matrices and dev.type == "cuda")
        self.master = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.grad = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.m = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.p16 = torch.zeros(self.n_decay, dtype=torch.bfloat16, device=dev) if self.bf16 else None
        for name, p, o, n in self.entries:
            self.master[o:o + n].copy_(p.detach().reshape(-1).float())
            gview = self.grad[o:o + n].view(p.shape)
            if self.bf16 and p.dim() >= 2:
                self.p16[o:o + n].copy_(p.detach().reshape(-1))
                p.data = self.p16[o:o + n].view(p.shape)
            else:
                p.data = self.master[o:o + n].view(p.shape)
            if dev.type == "cuda":
                p.main_grad = gview
            else:
                p.grad = gview
        self._scratch = torch.zeros(1024 + 8, dtype=torch.float32, device=dev)
        self._ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.skip_flag = torch.zeros(1, dtype=torch.int32, device=dev)

    # ------------------------------------------------------------------ helpers
    def zero_grad(self) -> None:
        self.grad.zero_()

    def named_master(self) -> Dict[str, torch.Tensor]:
        return {name: self.master[o:o + n].view(p.shape) for name, p, o, n in self.entries}

    def sync_compute_copy(self) -> None:
        """Refresh the bf16 compute copy from the fp32 masters (after loading weights)."""
        if self.bf16:
            self.p16.copy_(self.master[: self.n_decay])

    def load_master(self, name: str, value: torch.Tensor) -> None:
        for nm, p, o, n in self.entries:
            if nm == name:
                self.master[o:o + n].copy_(value.reshape(-1).to(self.master))
                if self.bf16 and p.dim() >= 2:
                    self.p16[o:o + n].copy_(self.master[o:o + n])
                return
        raise KeyError(name)

    def grad_norm(self, prescale: float = 1.0) -> torch.Tensor:
        """Global L2 norm of ``grad * prescale`` as a device scalar (no sync)."""
        if self.device.type == "cuda":
            nv.call("sumsq", nv.ptr(self.grad), nv.l(self.total), nv.ptr(self._scratch), nv.ptr(self._ticket),
                    nv.ptr(self.sumsq), nv.stream_ptr(self.device))
        else:
            self.sumsq[0] = (self.grad.double() ** 2).sum().float()
        return self.sumsq.sqrt() * prescale


class AdamW:
    """Fused AdamW over a :class:`FlatParams`."""

    def __init__(self, flat: FlatParams, lr: float, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1):
        self.flat, self.lr, self.betas, self.eps, self.wd = flat, lr, betas, eps, weight_decay
        self.step_count = 0

    def zero_grad(self) -> None:
        self.flat.zero_grad()

    def step(self, lr: Optional[float] = None, clip: float = 0.0, grad_prescale: float = 1.0) -> torch.Tensor:
        """Clip (global norm, on device) and update.  Returns the pre-clip gradient norm (device scalar)."""
        f = self.flat
        lr = self.lr if lr is None else lr
        self.step_count += 1
        norm = f.grad_norm(grad_prescale)
        b1, b2 = self.betas
        if f.device.type == "cuda":
            for lo, hi, wd in ((0, f.n_decay, self.wd), (f.n_decay, f.total, 0.0)):
                if hi <= lo:
                    continue
                p16 = f.p16[lo:hi] if (f.bf16 and hi <= f.n_decay) else None
                nv.call("adamw", nv.ptr(f.master[lo:hi]), nv.ptr(f.grad[lo:hi]), nv.ptr(f.m[lo:hi]), nv.ptr(f.v[lo:hi]),
                        nv.ptr(p16), nv.l(hi - lo), nv.f(lr), nv.f(b1), nv.f(b2), nv.f(self.eps), nv.f(wd),
                        nv.i(self.step_count), nv.f(grad_prescale), nv.f(clip), nv.ptr(f.sumsq), nv.ptr(f.skip_flag),
                        nv.stream_ptr(f.device))
        else:
            nrm = float(norm)
            if not math.isfinite(nrm):
                f.skip_flag[0] = 1
                return norm
            gs = grad_prescale * (min(1.0, clip / (nrm + 1e-6)) if clip > 0 else 1.0)
            g = f.grad * gs
            for lo, hi, wd in ((0, f.n_decay, self.wd), (f.n_decay, f.total, 0.0)):
                if hi > lo:
                    ref.adamw_step(f.master[lo:hi], g[lo:hi], f.m[lo:hi], f.v[lo:hi], self.step_count, lr, b1, b2, self.eps, wd)
        return norm

    def state_dict(self) -> Dict[str, torch.Tensor]:
        out = {"__step__": torch.tensor([self.step_count], dtype=torch.float32)}
        for name, p, o, n in self.flat.entries:
            out["m." + name] = self.flat.m[o:o + n].view(p.shape)
            out["v." + name] = self.flat.v[o:o + n].view(p.shape)
        return out

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        if "__step__" in sd:
            self.step_count = int(sd["__step__"].item())
        for name, p, o, n in self.flat.entries:
            if "m." + name in sd:
                self.flat.m[o:o + n].copy_(sd["m." + name].reshape(-1).to(self.flat.m))
                self.flat.v[o:o + n].copy_(sd["v." + name].reshape(-1).to(self.flat.v))
