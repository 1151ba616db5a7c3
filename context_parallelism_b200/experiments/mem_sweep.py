"""Memory-scaling sweep: largest sequence length before out-of-memory, and peak memory per length.

Runs a trainer in memory-probe mode (``CP_MEM_PROBE=1``) for growing T — doubling until a run fails, then
(optionally) bisecting between the last success and the first failure at a fixed granularity — each run
under a wall-clock timeout, with an ``nvidia-smi`` sampler recording the peak device usage, and classifies a
run as failed from its exit status and its log (out-of-memory / CUDA error / timeout).  Counterpart of the
reference's sweep scripts (Tests/mem_scaling_sweep.sh:93,195-229; Tests/bluscriptcp/mem_scaling_sweep*.sh);
the snapshots it leaves are turned into tables by ``mem_table.py``.

    python -m context_parallelism_b200.experiments.mem_sweep --trainer llama --nproc 8 --mode ulysses \
        --t-start 8192 --t-max 1048576 --bisect 4096 --out mem_runs
"""
from __future__ import annotations

import argparse
import os
import re
import subprocess
import sys
import threading
import time
from typing import Dict, Optional, Tuple

FAIL_PATTERNS = re.compile(r"out of memory|CUDA error|cudaErrorMemoryAllocation|OutOfMemoryError|symmetric heap exhausted|"
                           r"Traceback \(most recent call last\)|non-finite loss", re.I)


def is_fail(returncode: Optional[int], log_text: str) -> bool:
    return returncode is None or returncode != 0 or bool(FAIL_PATTERNS.search(log_text))


class SmiSampler:
    """Peak ``memory.used`` (MB, max over GPUs) while a run is alive."""

    def __init__(self, period_s: float = 0.5):
        self.period, self.peak, self._stop = period_s, 0, threading.Event()
        self.th = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "--query-gpu=memory.used", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=10).stdout.split()
                self.peak = max([self.peak] + [int(x) for x in out if x.isdigit()])
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        self.th.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self.th.join(timeout=5)


def run_one(args, T: int) -> Tuple[bool, int, str]:
    env = {k: v for k, v in os.environ.items()}
    env.update({"CP_MEM_PROBE": "1", "CP_MEM_PROBE_STEPS": str(args.steps), "CP_T": str(T), "CP_ATTN_MODE": args.mode,
                "CP_ROTATOR": args.rotator, "MEM_SNAPSHOT_DIR": args.out, "CP_MODEL_LABEL": args.label, "CP_SYNTHETIC": "1",
                "CP_LOG_DIR": args.out, "CP_B": str(args.batch)})
    for kv in args.env:
        k, v = kv.split("=", 1)
        env[k] = v
    module = f"context_parallelism_b200.trainers.{'gpt2_cp' if args.trainer == 'gpt2' else 'llama_cp'}"
    if args.nproc > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(args.port), "-m", module]
    else:
        cmd = [sys.executable, "-m", module]
    log_path = os.path.join(args.out, f"log_{args.label}_{args.mode}_T{T}_ws{args.nproc}.txt")
    rc: Optional[int] = None
    with SmiSampler() as smi, open(log_path, "w") as log:
        try:
            rc = subprocess.run(cmd, env=env, stdout=log, stderr=subprocess.STDOUT, timeout=args.timeout).returncode
        except subprocess.TimeoutExpired:
            log.write("\n[mem_sweep] TIMEOUT\n")
    text = open(log_path, errors="replace").read()
    return (not is_fail(rc, text)), smi.peak, log_path


def sweep(args) -> Dict[str, int]:
    os.makedirs(args.out, exist_ok=True)
    T, last_ok, first_fail = args.t_start, 0, 0
    rows = []
    while T <= args.t_max:
        ok, peak, log = run_one(args, T)
        rows.append((T, ok, peak))
        print(f"T={T} {'ok' if ok else 'FAIL'} peak_smi_mb={peak} log={log}", flush=True)
        if not ok:
            first_fail = T
            break
        last_ok, T = T, T * 2
    if first_fail and args.bisect > 0:
        lo, hi = last_ok, first_fail
        while hi - lo > args.bisect:
            mid = (lo + hi) // 2 // args.bisect * args.bisect
            if mid <= lo:
                break
            ok, peak, log = run_one(args, mid)
            rows.append((mid, ok, peak))
            print(f"T={mid} {'ok' if ok else 'FAIL'} peak_smi_mb={peak} (bisect)", flush=True)
            lo, hi = (mid, hi) if ok else (lo, mid)
        last_ok, first_fail = lo, hi
    with open(os.path.join(args.out, f"limits_{args.label}_{args.mode}_ws{args.nproc}.txt"), "w") as f:
        f.write(f"# label={args.label} mode={args.mode} rotator={args.rotator} ws={args.nproc} max_T_ok={last_ok} first_T_fail={first_fail}\n")
        for T, ok, peak in sorted(rows):
            f.write(f"{T},{int(ok)},{peak}\n")
    return {"max_T_ok": last_ok, "first_T_fail": first_fail}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--trainer", default="llama", choices=["llama", "gpt2"])
    ap.add_argument("--nproc", type=int, default=1)
    ap.add_argument("--mode", default="ulysses")
    ap.add_argument("--rotator", default="fused")
    ap.add_argument("--label", default="model")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--t-start", type=int, default=1024)
    ap.add_argument("--t-max", type=int, default=1 << 21)
    ap.add_argument("--bisect", type=int, default=0, help="granularity of the bisection after the first failure (0 = off)")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--timeout", type=float, default=1200.0)
    ap.add_argument("--port", type=int, default=29650)
    ap.add_argument("--out", default="mem_runs")
    ap.add_argument("--env", action="append", default=[], help="extra KEY=VALUE for the trainer (repeatable)")
    print(sweep(ap.parse_args(argv)))


if __name__ == "__main__":
    main()
