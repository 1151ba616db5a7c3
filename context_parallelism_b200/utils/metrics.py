"""Logging and observability: per-step log line, CSV with the reference's column sets, device-timed phase
timers, memory-probe snapshots, NVTX ranges.

CSV headers are the reference's (Scripts/Blutrain/gpt2_cp_test.cpp:1117-1120 for GPT-2 with per-layer timers;
bluscriptCP.cpp:1147-1148 for Llama).  Unlike the reference's ``CudaTimer``, which synchronises the device at
every read and so perturbs overlap (gpt2_cp_test.cpp:53-72), ``PhaseTimers`` records CUDA events without
synchronising and resolves them once per step.
"""
from __future__ import annotations

import contextlib
import os
import subprocess
import time
from typing import Dict, List, Optional

import torch

GPT2_CSV = ("step,loss,val_loss,lr,grad_norm,dt_ms,tok_per_sec,timer_data,timer_fwd,timer_loss,timer_bwd,timer_clip,"
            "timer_optim,timer_tok_emb,timer_pos_emb,timer_attn_cp,timer_mlp,timer_ln_f,timer_lm_head,mem_gpu_mb")
LLAMA_CSV = "step,loss,val_loss,lr,grad_norm,dt_ms,tok_per_sec,timer_data,timer_fwd,timer_loss,timer_bwd,timer_clip,timer_optim,mem_gpu_mb"


def is_master() -> bool:
    return int(os.environ.get("RANK", "0")) == 0


def log(msg: str) -> None:
    """Rank-0 only notice (the reference gates on OMPI_COMM_WORLD_RANK / PMI_RANK, context_parallel/CPLog.h:11-17)."""
    if is_master():
        print(msg, flush=True)


@contextlib.contextmanager
def nvtx(name: str):
    """NVTX range (the reference's EmitNVTX / nvtxRangePushA markers, gpt2_cp_test.cpp:21-26)."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class PhaseTimers:
    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"
        self.device = device
        self._open: Dict[str, object] = {}
        self._pairs: List[tuple] = []
        self.ms: Dict[str, float] = {}

    @contextlib.contextmanager
    def phase(self, name: str):
        with nvtx(name):
            if self.cuda:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                try:
                    yield
                finally:
                    b.record()
                    self._pairs.append((name, a, b))
            else:
                t0 = time.perf_counter()
                try:
                    yield
                finally:
                    self.ms[name] = self.ms.get(name, 0.0) + (time.perf_counter() - t0) * 1e3

    def resolve(self) -> Dict[str, float]:
        """Synchronise once and return accumulated milliseconds per phase; resets the timers."""
        if self.cuda and self._pairs:
            torch.cuda.synchronize(self.device)
            for name, a, b in self._pairs:
                self.ms[name] = self.ms.get(name, 0.0) + a.elapsed_time(b)
            self._pairs = []
        out, self.ms = self.ms, {}
        return out


def gpu_mem_mb(device: torch.device) -> float:
    if device.type != "cuda":
        return 0.0
    free, total = torch.cuda.mem_get_info(device)
    return (total - free) / 2 ** 20


class CsvLog:
    def __init__(self, path: str, header: str, resumed: bool = False, resume_note: str = ""):
        self.path, self.cols = path, header.split(",")
        self.enabled = is_master()
        if not self.enabled:
            return
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        if resumed and os.path.exists(path):
            with open(path, "a") as f:
                f.write(f"# resumed {resume_note}\n")
        else:
            with open(path, "w") as f:
                f.write(header + "\n")

    def row(self, **kw) -> None:
        if not self.enabled:
            return
        vals = []
        for c in self.cols:
            v = kw.get(c, "")
            vals.append(f"{v:.6g}" if isinstance(v, float) else str(v))
        with open(self.path, "a") as f:
            f.write(",".join(vals) + "\n")


def step_line(step: int, max_steps: int, loss: float, lr: float, norm: float, dt_ms: float, tok_s: float, mem_mb: float) -> str:
    left = (max_steps - step - 1) * dt_ms / 1e3
    return (f"step {step:5d} | loss {loss:.6f} | lr {lr:.4e} | norm {norm:.4f} | dt {dt_ms:.2f}ms | "
            f"tok/sec {tok_s:.1f} | mem {mem_mb:.0f}MB | Time Left {int(left // 3600)}h{int(left % 3600 // 60):02d}m")


def write_mem_snapshot(path: str, cfg, impl: str, rotator: str, device: torch.device, extra: Optional[Dict[str, object]] = None) -> None:
    """Memory-probe snapshot in the ``# key=value`` header format the sweep/table tools parse
    (gpt2_cp_test.cpp:1806-1873): device usage from the driver, allocator statistics, nvidia-smi per GPU."""
    lines = [f"# impl={impl} label={cfg.model_label} rotator={rotator} attn_mode={cfg.attn_mode} T={cfg.T} B={cfg.B} "
             f"world_size={cfg.world_size} cp_size={cfg.cp_size} n_embd={cfg.n_embd} n_layer={cfg.n_layer} n_head={cfg.n_head} "
             f"n_kv_head={cfg.n_kv_head} dtype={cfg.dtype} recompute={cfg.recompute}"]
    if device.type == "cuda":
        free, total = torch.cuda.mem_get_info(device)
        st = torch.cuda.memory_stats(device)
        lines.append(f"# CUDA_MEMGETINFO_USED_MB={(total - free) / 2 ** 20:.0f} TOTAL_MB={total / 2 ** 20:.0f}")
        lines.append(f"# ALLOC reserved_mb={st.get('reserved_bytes.all.current', 0) / 2 ** 20:.0f} "
                     f"active_mb={st.get('active_bytes.all.current', 0) / 2 ** 20:.0f}")
        res_pk, act_pk = st.get("reserved_bytes.all.peak", 0), st.get("active_bytes.all.peak", 0)
        frag = 100.0 * (res_pk - act_pk) / res_pk if res_pk else 0.0
        lines.append(f"# ALLOC_PEAK reserved_mb={res_pk / 2 ** 20:.0f} active_mb={act_pk / 2 ** 20:.0f} internal_frag_pct={frag:.2f}")
        try:
            out = subprocess.run(["nvidia-smi", "--query-gpu=memory.used", "--format=csv,noheader,nounits"],
                                 capture_output=True, text=True, timeout=10).stdout.split()
            lines.append("# SMI_USED_MB_PER_GPU=" + ",".join(out))
        except Exception:
            lines.append("# SMI_USED_MB_PER_GPU=unavailable")
    for k, v in (extra or {}).items():
        lines.append(f"# {k}={v}")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
