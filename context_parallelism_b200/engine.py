"""Training engine: the public API a user (and ``bench.py``) drives.

``TrainEngine(cfg)`` builds the device mesh, the context-parallel context, the model, the flat
parameter store, the fused AdamW and the bucketed gradient reducer.  ``train_step(tokens, targets)``
takes FULL sequences ``[B, T]`` (pinned host or device int64), copies them to the device, gathers the
local shard with the same permutation for inputs and targets, and runs forward, backward, gradient
all-reduce (AVERAGE over all dp·cp ranks) and the optimiser step.  It returns the mean loss of the
local shard as a device scalar; ``global_loss`` averages it over ranks.  This is the step of the
reference trainers (Scripts/Blutrain/bluscriptCP.cpp:1653-1785, gpt2_cp_test.cpp:1497-1763).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .config import Config
from .ops import permute
from .ops.optim import AdamW, FlatParams
from .parallel.cp_attention import CPContext
from .parallel.ddp import GradReducer
from .parallel.mesh import DeviceMesh
from .utils.lr import cosine_lr, rewarmup_lr


class TrainEngine:
    def __init__(self, cfg: Config, device: Optional[torch.device] = None, mesh: Optional[DeviceMesh] = None,
                 standalone: bool = False):
        """``standalone=True`` builds a single-process engine (world size 1) even inside a distributed job; the
        parity tests use it for the unsharded reference run."""
        cfg.validate()
        self.cfg = cfg
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = device
        self.rank = dist.get_rank() if (dist.is_initialized() and not standalone) else 0
        self.world = dist.get_world_size() if (dist.is_initialized() and not standalone) else 1
        if cfg.world_size != self.world:
            raise ValueError(f"config world_size={cfg.world_size} but the job has {self.world} ranks")
        self.mesh = mesh or DeviceMesh.for_config(cfg, self.rank, self.world, create_groups=not standalone)
        self.cp = CPContext.from_mesh(cfg, self.mesh)
        if device.type == "cuda" and self.cp.cp_size > 1 and cfg.rotator == "fused":
            from .parallel.fused import FusedComm
            self.cp.fused = FusedComm.create(cfg, self.cp, device)
        self.native_pg = None
        import os
        if (device.type == "cuda" and self.cp.ring_size > 1 and cfg.rotator == "p2p" and self.cp.ring_group is not None
                and os.environ.get("CP_NATIVE_PG", "1") != "0"):
            # the NCCL baseline ring hops through the native process group: a communicator and a stream of its own
            from .parallel import rotators
            from .parallel.process_group import NativeProcessGroup
            self.native_pg = NativeProcessGroup.create(self.cp.ring_group, cfg.watchdog_s, True, device)
            rotators.NATIVE_GROUPS[id(self.cp.ring_group)] = self.native_pg
        if cfg.family == "gpt2":
            from .models.gpt2 import GPT2
            self.model = GPT2(cfg, self.cp, device)
        else:
            from .models.llama import Llama
            self.model = Llama(cfg, self.cp, device)
        if device.type == "cuda":
            from .ops import attention as _A
            _A.FP32_ACCURATE = bool(cfg.attn_fp32)
            if cfg.attn_fp32 and self.cp.cp_size > 1 and not (cfg.attn_mode == "ulysses" and cfg.rotator != "fused"):
                raise ValueError("ATTN_FP32=1 (fp32-accurate attention for parity runs) is supported on one GPU and for Ulysses "
                                 "with an NCCL rotator (CP_ROTATOR=alltoall); the other paths are built on the tensor-core kernels")
        bf16 = cfg.dtype == "bf16" and device.type == "cuda"
        if device.type == "cuda" and not bf16:
            raise ValueError("the CUDA kernels compute in bf16; CP_DTYPE=fp32 is the CPU oracle path")
        if self.world > 1:
            # every replica starts from rank 0's values (DDP ``init_sync``, bluscriptCP.cpp:1011)
            with torch.no_grad():
                for p in self.model.parameters():
                    dist.broadcast(p.data, 0)
        fused_world = self.cp.fused if (self.cp.fused is not None and self.cp.fused.covers_world()) else None
        shard = fused_world if (cfg.shard_optim and not cfg.no_grad_allreduce) else None
        self.flat = FlatParams(self.model.named_parameters(), bf16, cfg.grad_bucket_mb, shard)
        self.opt = AdamW(self.flat, cfg.max_lr, (cfg.beta1, cfg.beta2), cfg.adam_eps, cfg.weight_decay)
        fused_ar = fused_world.grad_allreduce_for(self.flat) if fused_world is not None else None
        self.reducer = GradReducer(self.flat, None, self.world, cfg.grad_bucket_mb, fused_ar,
                                   overlap=not (cfg.debug.no_overlap or cfg.debug.no_overlap_bwd))
        if cfg.no_grad_allreduce:
            self.reducer.enabled = False
        self.step_idx = 0
        self.resume_anchor = -1
        self._pos_dev = {}
        self.last_grad_norm: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ helpers
    def lr_at(self, step: int) -> float:
        c = self.cfg
        anchor = c.rewarmup_anchor if c.rewarmup_anchor >= 0 else self.resume_anchor
        if c.rewarmup_steps > 0 and anchor >= 0:
            return rewarmup_lr(step, c.max_lr, c.min_lr, c.warmup_steps, c.max_steps, anchor, c.rewarmup_steps, c.rewarmup_peak)
        return cosine_lr(step, c.max_lr, c.min_lr, c.warmup_steps, c.max_steps)

    def local_pos(self, T: int) -> torch.Tensor:
        p = self._pos_dev.get(T)
        if p is None:
            p = self._pos_dev[T] = self.cp.local_positions(T).to(self.device)
        return p

    def shard_batch(self, tokens: torch.Tensor, targets: Optional[torch.Tensor]):
        """Full ``[B, T]`` (host or device) → local ``[B, T/cp]`` on the device, plus positions."""
        tokens = tokens.to(self.device, non_blocking=True)
        if targets is not None:
            targets = targets.to(self.device, non_blocking=True)
        pos = self.local_pos(tokens.shape[1])
        if self.cp.cp_size == 1:
            return tokens, targets, pos
        return (permute.gather_tokens(tokens, pos),
                permute.gather_tokens(targets, pos) if targets is not None else None, pos)

    # ------------------------------------------------------------------ one optimiser step
    def forward_backward(self, tokens, targets, accum: int = 1, last: bool = True) -> torch.Tensor:
        idx, tgt, pos = self.shard_batch(tokens, targets)
        n_local = idx.numel()
        scale = 1.0 / (n_local * accum)
        self.reducer.begin_backward()
        ctx = self.reducer.no_sync() if not last else _null()
        with ctx:
            loss_sum = self.model.loss_sum(idx, tgt, pos, scale)
            loss_sum.backward(torch.tensor(scale, device=loss_sum.device, dtype=loss_sum.dtype))
        if last:
            self.reducer.finish()
        return loss_sum.detach() / n_local

    def optimizer_step(self) -> torch.Tensor:
        lr = self.lr_at(self.step_idx)
        norm = self.opt.step(lr, self.cfg.grad_clip)
        self.opt.zero_grad()
        self.step_idx += 1
        self.last_grad_norm = norm
        return norm

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        loss = self.forward_backward(tokens, targets, 1, True)
        self.optimizer_step()
        return loss

    def global_loss(self, local_loss: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return local_loss
        t = local_loss.detach().clone().float().reshape(1)
        dist.all_reduce(t)
        return (t / self.world).squeeze(0)

    @torch.no_grad()
    def eval_loss(self, tokens, targets) -> torch.Tensor:
        idx, tgt, pos = self.shard_batch(tokens, targets)
        return self.model.loss_sum(idx, tgt, pos, 0.0) / idx.numel()

    def finish_step(self) -> None:
        """Host-side end of a step's device work, called by the trainers before the optimiser runs: wait for the
        stream with the ``CP_WATCHDOG_S`` deadline (a polling wait on a watched work handle, so a stuck collective
        raises ``StepTimeout`` instead of hanging the job), then turn any bounded-wait expiry or bounds failure the
        kernels reported into an exception, so that an update is never applied on top of stale data."""
        if self.device.type == "cuda":
            from .parallel.work import wait_for_stream
            wait_for_stream(self.device, self.cfg.watchdog_s, f"step {self.step_idx}")
        self.check_kernels()

    def check_kernels(self) -> None:
        """Raise if any kernel reported a bounded-wait expiry or a bounds failure (one small D2H read)."""
        if self.device.type == "cuda":
            from . import _native as nv
            nv.status_for(self.device).check("train step")

    def close(self) -> None:
        if self.native_pg is not None:
            from .parallel import rotators
            torch.cuda.synchronize(self.device)
            rotators.NATIVE_GROUPS.pop(id(self.cp.ring_group), None)
            self.native_pg.close()
            self.native_pg = None
        if self.cp.fused is not None:
            self.cp.fused.close()
            self.cp.fused = None


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
