"""Run the configurations the reference published numbers for, through the two trainers, and report tokens/s the
way the reference does (wall clock of whole optimiser steps on rank 0, warm-up steps dropped).

* ``gpt2_44m``  – GPT-2 44M (n_embd 384, 3 layers, 6 heads), B = 4, T = 1024, global batch 65 536 tokens (16 micro
  batches per step), world size 2, Ulysses or ring: 70 000 tok/s (C++ Ulysses) and 62 152 tok/s (PyTorch ring) on
  2x RTX 3060 in the reference's notebook (graph.ipynb:43-70).
* ``llama_48m`` – Llama-style 48M (d 384, 6 layers, 6/2 heads, head_dim 64), T = 4096, B = 2, global batch 524 288
  tokens, one GPU: about 43 000 tok/s on an RTX 6000 Ada (comparison_curve.png).

Synthetic uniform-random tokens stand in for the dataset (throughput does not depend on the token values).

    python -m context_parallelism_b200.experiments.published_configs --which gpt2_44m --mode ulysses --nproc 2
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys

CONFIGS = {
    "gpt2_44m": dict(module="context_parallelism_b200.trainers.gpt2_cp", published={"ulysses": 70000.0, "ring": 62152.0},
                     env={"CP_MODEL_44M": "1", "CP_B": "4", "CP_T": "1024", "CP_GLOBAL_BATCH": "65536", "CP_WEIGHT_TYING": "1"}),
    "llama_48m": dict(module="context_parallelism_b200.trainers.llama_cp", published={"ulysses": 43000.0, "ring": 43000.0},
                      env={"CP_N_EMBD": "384", "CP_N_LAYER": "6", "CP_N_HEAD": "6", "CP_N_KVHEAD": "2", "CP_B": "2", "CP_T": "4096",
                           "CP_GLOBAL_BATCH": "524288"}),
}
_STEP = re.compile(r"^step\s+(\d+) \|.*dt\s+([0-9.]+)ms \| tok/sec\s+([0-9.]+)")


def run(which: str, mode: str, nproc: int, steps: int, skip: int, port: int, extra_env=None) -> dict:
    c = CONFIGS[which]
    env = dict(os.environ, **c["env"], CP_ATTN_MODE=mode, CP_MAX_STEPS=str(steps), CP_SYNTHETIC="1", CP_CKPT="0", CP_VAL_FREQ="0",
               CP_WARMUP="2", **(extra_env or {}))
    cmd = [sys.executable, "-m", c["module"]] if nproc == 1 else [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
        "--master-port", str(port), "-m", c["module"]]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True)
    rows = [m for m in (_STEP.match(ln) for ln in r.stdout.splitlines()) if m]
    timed = [(float(m.group(2)), float(m.group(3))) for m in rows if int(m.group(1)) >= skip]
    out = {"config": which, "mode": mode, "world_size": nproc, "steps_timed": len(timed), "returncode": r.returncode,
           "published_tok_per_sec": c["published"].get(mode)}
    if timed:
        out["ms_per_step"] = sum(t for t, _ in timed) / len(timed)
        out["tok_per_sec"] = sum(v for _, v in timed) / len(timed)
        out["vs_published"] = out["tok_per_sec"] / c["published"][mode] if c["published"].get(mode) else None
    else:
        out["stderr_tail"] = r.stderr[-1500:]
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--which", choices=sorted(CONFIGS), required=True)
    ap.add_argument("--mode", default="ulysses", choices=["ulysses", "ring"])
    ap.add_argument("--nproc", type=int, default=1)
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--skip", type=int, default=3, help="leading steps left out of the average")
    ap.add_argument("--port", type=int, default=29671)
    a = ap.parse_args(argv)
    print(json.dumps(run(a.which, a.mode, a.nproc, a.steps, a.skip, a.port)))


if __name__ == "__main__":
    main()
