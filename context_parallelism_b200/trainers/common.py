"""Shared training loop of the two trainers: run numbering and auto-resume, data loaders with
fast-forward, gradient accumulation, validation, checkpointing, CSV/log output, memory-probe mode and the
NaN/Inf guard (Scripts/Blutrain/bluscriptCP.cpp:1042-1192,1653-1888; gpt2_cp_test.cpp:985-1235,1497-1881)."""
from __future__ import annotations

import math
import os
import time
from typing import Callable, Optional

import torch
import torch.distributed as dist

from ..config import Config
from ..engine import TrainEngine
from ..utils import ckpt as ckpt_mod
from ..utils import data as data_mod
from ..utils import metrics as M


def broadcast_ints(vals, src: int = 0):
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return list(vals)
    backend = dist.get_backend()
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    t = torch.tensor(list(vals), dtype=torch.int64, device=dev)
    dist.broadcast(t, src)
    return [int(x) for x in t.tolist()]


def all_reduce_mean(x: float) -> float:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return x
    backend = dist.get_backend()
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    t = torch.tensor([x], dtype=torch.float64, device=dev)
    dist.all_reduce(t)
    return float(t.item()) / dist.get_world_size()


def train(cfg: Config, eng: TrainEngine, impl: str, csv_header: str,
          on_step_begin: Optional[Callable[[int], None]] = None,
          periodic: Optional[Callable[[int], None]] = None) -> None:
    dev, rank = eng.device, eng.rank
    dp_rank, dp_size = eng.cp.dp_rank, eng.cp.dp_size
    accum = 1 if cfg.mem_probe else cfg.grad_accum
    max_steps = cfg.mem_probe_steps if cfg.mem_probe else cfg.max_steps
    train_ld = data_mod.make_loader(cfg, "train", dp_rank, dp_size)
    val_ld = data_mod.make_loader(cfg, "val", dp_rank, dp_size)

    # ---- run number / resume: decided on rank 0, broadcast so every rank builds the same names
    mgr = ckpt_mod.CheckpointManager(cfg.ckpt_dir, cfg.ckpt_prefix, cfg.ckpt_keep, rank)
    run, resuming = 0, False
    use_ckpt = cfg.checkpointing and not cfg.mem_probe
    if rank == 0 and (use_ckpt or cfg.ckpt_resume >= 0):
        run, resuming = mgr.resolve_run(cfg.max_steps, cfg.ckpt_new_run, cfg.ckpt_resume)
    run, resuming = broadcast_ints([run, int(resuming)])
    start_step, last_loss = 0, float("nan")
    if resuming:
        start_step, last_loss = mgr.load_latest(run, eng.model, eng.flat, eng.opt)
        eng.step_idx = start_step
        eng.resume_anchor = start_step
        train_ld.skip_batches(start_step * accum)          # same data order as an uninterrupted run
        M.log(f"[resume] run {run} from step {start_step} (loss {last_loss:.4f})")
    log_path = os.path.join(cfg.log_dir, f"{cfg.ckpt_prefix}_run{run}_log.csv")
    csv = M.CsvLog(log_path, csv_header, resumed=resuming, resume_note=f"from step {start_step}")
    if rank == 0 and not cfg.mem_probe:
        os.makedirs(cfg.log_dir, exist_ok=True)
        with open(os.path.join(cfg.log_dir, f"{cfg.ckpt_prefix}_run{run}_config.txt"), "w") as f:
            f.write(cfg.describe() + "\n")
    timers = M.PhaseTimers(dev)
    alloc_csv = None
    if cfg.alloc_csv and rank == 0:
        # CP_ALLOC_CSV: one row of caching-allocator statistics per step (gpt2_cp_test.cpp:1802)
        os.makedirs(os.path.dirname(os.path.abspath(cfg.alloc_csv)), exist_ok=True)
        alloc_csv = open(cfg.alloc_csv, "a" if resuming else "w")
        if not resuming:
            alloc_csv.write("step,allocated_mb,reserved_mb,peak_allocated_mb,peak_reserved_mb,num_alloc_retries,driver_used_mb\n")
    tokens_per_step = cfg.B * cfg.T * dp_size * accum
    val_loss = float("nan")
    M.log(f"[{impl}] world={cfg.world_size} dp={dp_size} cp={cfg.cp_size} mode={cfg.attn_mode} rotator={cfg.rotator} "
          f"T={cfg.T} B={cfg.B} accum={accum} tokens/step={tokens_per_step} steps={start_step}->{max_steps}")

    for step in range(start_step, max_steps):
        t0 = time.perf_counter()
        if on_step_begin is not None:
            on_step_begin(step)
        if not cfg.mem_probe and cfg.val_freq > 0 and step % cfg.val_freq == 0:
            tot = 0.0
            for _ in range(cfg.val_steps):
                x, y = val_ld.next_batch()
                tot += float(eng.global_loss(eng.eval_loss(x, y)))
            val_loss = tot / max(1, cfg.val_steps)
            M.log(f"validation loss {val_loss:.4f}")
        if periodic is not None:
            periodic(step)
        loss_acc = torch.zeros((), dtype=torch.float32, device=dev)
        for micro in range(accum):
            with timers.phase("timer_data"):
                x, y = train_ld.next_batch()
            with timers.phase("timer_fwd_bwd"):
                loss_acc += eng.forward_backward(x, y, accum, last=(micro == accum - 1)).float() / accum
        lr = eng.lr_at(eng.step_idx)
        eng.finish_step()          # bounded wait + kernel status: a failed step never reaches the optimiser
        with timers.phase("timer_optim"):
            norm = eng.optimizer_step()
        loss = float(eng.global_loss(loss_acc))
        eng.check_kernels()
        if not math.isfinite(loss):
            # the reference aborts the job (bluscriptCP.cpp:1730-1733); the update itself was already skipped on
            # the device by the non-finite-norm guard of the fused optimiser
            raise RuntimeError(f"non-finite loss {loss} at step {step}")
        ph = timers.resolve()
        dt_ms = (time.perf_counter() - t0) * 1e3
        tok_s = tokens_per_step / (dt_ms / 1e3)
        mem = M.gpu_mem_mb(dev)
        M.log(M.step_line(step, max_steps, loss, lr, float(norm), dt_ms, tok_s, mem))
        csv.row(step=step, loss=loss, val_loss=val_loss, lr=lr, grad_norm=float(norm), dt_ms=dt_ms, tok_per_sec=tok_s,
                timer_data=ph.get("timer_data", 0.0), timer_fwd=ph.get("timer_fwd_bwd", 0.0), timer_optim=ph.get("timer_optim", 0.0),
                mem_gpu_mb=mem)
        if alloc_csv is not None:
            st = torch.cuda.memory_stats(dev) if dev.type == "cuda" else {}
            mb = lambda k: st.get(k, 0) / 2 ** 20          # noqa: E731
            alloc_csv.write(f"{step},{mb('allocated_bytes.all.current'):.1f},{mb('reserved_bytes.all.current'):.1f},"
                            f"{mb('allocated_bytes.all.peak'):.1f},{mb('reserved_bytes.all.peak'):.1f},{st.get('num_alloc_retries', 0)},{mem:.0f}\n")
            alloc_csv.flush()
        if cfg.debug.dump_fwd and step == start_step:
            # DUMP_FWD: the first step's forward result for cross-implementation parity (loss and final hidden state)
            with torch.no_grad():
                idx, _, pos = eng.shard_batch(x, None)
                hdn = eng.model.hidden(idx, pos)
            from ..utils.debug import DebugTools
            DebugTools(cfg, rank).dump(True, "fwd", step, hidden=hdn, loss=torch.tensor([loss]), positions=pos.float())
        last_loss = loss
        if use_ckpt and ((step + 1) % cfg.ckpt_freq == 0 or step + 1 == max_steps):
            mgr.save(run, step + 1, eng.model, eng.flat, eng.opt, loss)
    if cfg.mem_probe:
        label = f"{impl}_{cfg.model_label}_{cfg.rotator if cfg.attn_mode != 'ulysses' else 'ulysses'}_T{cfg.T}_ws{cfg.world_size}"
        path = os.path.join(cfg.mem_snapshot_dir, label + ".txt")
        if rank == 0:
            M.write_mem_snapshot(path, cfg, impl, cfg.rotator, dev, {"final_loss": last_loss})
        M.log(f"[mem-probe] snapshot {path}")
    if alloc_csv is not None:
        alloc_csv.close()
    train_ld.close()
    val_ld.close()
