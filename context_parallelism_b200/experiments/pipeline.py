"""Resumable search → fine-tune → eval pipelines for context extension.

What the reference drives with shell scripts (Tests/bluscriptcp/run_longrope_pipeline.sh, longrope_progressive.sh,
longrope_autorun.sh, alt_pos_sweep.sh) as one Python tool:

* ``progressive`` – for every extension factor in ``--stages`` (from the base length): (1) GA search of LongRoPE factors
  on the CURRENT checkpoint with the resident evaluator, (2) fine-tune at that length with the searched cache installed
  and the two-stage LR re-warm-up, (3) per-position perplexity at that length.  The fine-tuned checkpoint of a stage is
  the base of the next.
* ``altpos``      – fine-tune + eval once per position-relabelling scheme (``cream``, ``pose``, ``randpos``).

Every sub-step leaves ``<state_dir>/<name>.done`` (written atomically, holding the step's result as JSON) and is skipped
when the marker exists, so the same command continues where a killed run stopped; a half-done fine-tune resumes from
its newest checkpoint through the trainer's own auto-resume, a half-done search from its saved population and memo.
``--wait-idle-mb`` polls ``nvidia-smi`` (read-only) until every chosen GPU uses less than that much memory before
anything is launched.

    python -m context_parallelism_b200.experiments.pipeline progressive --stages 2 4 --base-t 4096 --nproc 8 \
        --env CP_ATTN_MODE=ring --env CP_DATA_ROOT=/data ...
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from typing import Callable, Dict, List, Optional

from ..utils.ckpt import CheckpointManager
from . import longrope_search as LS

TRAINER = "context_parallelism_b200.trainers.llama_cp"


class Steps:
    """``.done`` markers: ``run(name, fn)`` calls ``fn`` unless ``<dir>/<name>.done`` exists and returns its result."""

    def __init__(self, state_dir: str):
        self.dir = state_dir
        os.makedirs(state_dir, exist_ok=True)
        self.skipped: List[str] = []
        self.ran: List[str] = []

    def path(self, name: str) -> str:
        return os.path.join(self.dir, name + ".done")

    def done(self, name: str) -> bool:
        return os.path.exists(self.path(name))

    def run(self, name: str, fn: Callable[[], Optional[dict]]) -> dict:
        if self.done(name):
            self.skipped.append(name)
            print(f"[pipeline] {name}: done already, skipped", flush=True)
            with open(self.path(name)) as f:
                return json.load(f)
        print(f"[pipeline] {name}: start", flush=True)
        t0 = time.time()
        res = dict(fn() or {})
        res["seconds"] = round(time.time() - t0, 2)
        tmp = self.path(name) + ".tmp"
        with open(tmp, "w") as f:
            json.dump(res, f)
        os.replace(tmp, self.path(name))                    # the marker appears only after the step succeeded
        self.ran.append(name)
        return res


def launch_cmd(nproc: int, port: int, module: str = TRAINER) -> List[str]:
    if nproc == 1:
        return [sys.executable, "-m", module]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
            "--master-port", str(port), "-m", module]


def run_trainer(env: Dict[str, str], nproc: int, port: int, log_path: str, timeout: Optional[float] = None) -> str:
    e = dict(os.environ, **{k: str(v) for k, v in env.items()})
    r = subprocess.run(launch_cmd(nproc, port), env=e, capture_output=True, text=True, timeout=timeout)
    with open(log_path, "w") as f:
        f.write(r.stdout + "\n--- stderr\n" + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"trainer failed (rc {r.returncode}); see {log_path}\n{r.stderr[-1500:]}")
    return r.stdout


def wait_for_idle_gpus(max_used_mb: int, gpus: Optional[List[int]] = None, poll_s: float = 30.0, max_wait_s: float = 0.0,
                       query: Optional[Callable[[], List[int]]] = None) -> bool:
    """Poll until every chosen GPU uses less than ``max_used_mb`` MB (the reference's autorun waits for a free box the
    same way, longrope_autorun.sh:45-82).  ``query`` returns used MB per GPU (default: ``nvidia-smi``, read-only).
    Returns False if ``max_wait_s`` (when > 0) ran out."""
    def smi() -> List[int]:
        out = subprocess.run(["nvidia-smi", "--query-gpu=memory.used", "--format=csv,noheader,nounits"], capture_output=True, text=True).stdout
        return [int(x) for x in out.split() if x.strip().isdigit()]
    query = query or smi
    t0 = time.time()
    while True:
        used = query()
        sel = [used[i] for i in gpus] if gpus else used
        if sel and all(u < max_used_mb for u in sel):
            return True
        if max_wait_s > 0 and time.time() - t0 > max_wait_s:
            return False
        time.sleep(poll_s)


def _env_list(items: List[str]) -> Dict[str, str]:
    out = {}
    for it in items:
        k, _, v = it.partition("=")
        out[k] = v
    return out


def progressive(a) -> dict:
    steps = Steps(a.state_dir)
    base_env = dict(_env_list(a.env), CP_CKPT="1", CP_CKPT_DIR=a.ckpt_dir, CP_LOG_DIR=a.state_dir)
    run = a.base_run
    summary = {"stages": []}
    for i, s in enumerate(a.stages):
        T = a.base_t * s
        tag = f"s{s}"
        fac = os.path.join(a.state_dir, f"factors_{tag}.txt")

        def do_search(T=T, s=s, tag=tag, fac=fac, run=run):
            ns = argparse.Namespace(head_dim=a.head_dim, scale=float(s), orig_len=a.base_t, base=a.rope_base, n_hat=0,
                                    population=a.population, generations=a.generations, pool=a.pool, seed=a.seed,
                                    workdir=os.path.join(a.state_dir, f"search_{tag}"), fresh=False)
            env = dict(base_env, CP_T=str(T), CP_B="1", CP_CKPT_RESUME=str(run), CP_EVAL_WINDOWS=str(a.search_windows))
            os.environ.update({k: str(v) for k, v in env.items()})          # the evaluator workers inherit the stage's settings
            best, val = LS.search(ns, launch_cmd(a.search_nproc, a.port + 50))
            LS.write_factors(fac, best, 0, s, T)
            return {"best_ppl": val, "factors": fac}

        def do_finetune(T=T, s=s, tag=tag, fac=fac, run=run, i=i):
            ft_run = a.ft_run_base + i
            # the stage's run starts as a copy of the previous run's newest checkpoint; resuming it continues from there
            # (and a killed fine-tune resumes from its own newest checkpoint)
            start = CheckpointManager(a.ckpt_dir, a.prefix).seed_run_from(run, ft_run)
            base_step = CheckpointManager(a.ckpt_dir, a.prefix).list_runs()[run][-1]
            env = dict(base_env, CP_T=str(T), CP_B=str(a.ft_batch), CP_GLOBAL_BATCH=str(a.ft_batch * T), CP_LONGROPE_FACTORS=fac,
                       CP_REWARMUP=str(a.rewarmup), CP_REWARMUP_ANCHOR=str(base_step), CP_MAX_STEPS=str(base_step + a.ft_steps),
                       CP_CKPT_FREQ=str(a.ckpt_freq), CP_CKPT_RESUME=str(ft_run), CP_VAL_FREQ="0")
            del start
            out = run_trainer(env, a.nproc, a.port, os.path.join(a.state_dir, f"finetune_{tag}.log"), a.timeout)
            last = [ln for ln in out.splitlines() if ln.startswith("step")]
            return {"run": ft_run, "last_step_line": last[-1] if last else ""}

        def do_eval(T=T, tag=tag, fac=fac, i=i):
            csv = os.path.join(a.state_dir, f"ppl_prog_{tag}.csv")
            env = dict(base_env, CP_T=str(T), CP_B="1", CP_LONGROPE_FACTORS=fac, CP_EVAL_PPL="1", CP_EVAL_WINDOWS=str(a.eval_windows),
                       CP_EVAL_OUT=csv, CP_CKPT_RESUME=str(a.ft_run_base + i))
            out = run_trainer(env, a.nproc, a.port + 1, os.path.join(a.state_dir, f"eval_{tag}.log"), a.timeout)
            ppl = [ln for ln in out.splitlines() if "PPL" in ln]
            return {"csv": csv, "ppl_line": ppl[-1] if ppl else ""}
        st = {"factor": s, "T": T, "search": steps.run(f"search_{tag}", do_search), "finetune": steps.run(f"finetune_{tag}", do_finetune),
              "eval": steps.run(f"eval_{tag}", do_eval)}
        summary["stages"].append(st)
        run = a.ft_run_base + i
    summary["ran"], summary["skipped"] = steps.ran, steps.skipped
    return summary


def altpos(a) -> dict:
    steps = Steps(a.state_dir)
    base_env = dict(_env_list(a.env), CP_CKPT="1", CP_CKPT_DIR=a.ckpt_dir, CP_LOG_DIR=a.state_dir, CP_T=str(a.base_t))
    out = {"modes": []}
    for i, mode in enumerate(a.modes):
        def ft(mode=mode, i=i):
            mgr = CheckpointManager(a.ckpt_dir, a.prefix)
            mgr.seed_run_from(a.base_run, a.ft_run_base + i)
            base_step = mgr.list_runs()[a.base_run][-1]
            env = dict(base_env, CP_CREAM_MODE=mode, YARN_SCALE=str(a.yarn_scale), YARN_ORIG_MAXPOS=str(a.base_t),
                       CP_MAX_STEPS=str(base_step + a.ft_steps), CP_CKPT_FREQ=str(a.ckpt_freq), CP_CKPT_RESUME=str(a.ft_run_base + i),
                       CP_VAL_FREQ="0")
            o = run_trainer(env, 1, a.port, os.path.join(a.state_dir, f"altpos_{mode}.log"), a.timeout)   # relabelling needs CP_SIZE=1
            last = [ln for ln in o.splitlines() if ln.startswith("step")]
            return {"last_step_line": last[-1] if last else ""}

        def ev(mode=mode, i=i):
            csv = os.path.join(a.state_dir, f"ppl_{mode}.csv")
            env = dict(base_env, CP_T=str(int(a.base_t * a.yarn_scale)), YARN_SCALE=str(a.yarn_scale), YARN_ORIG_MAXPOS=str(a.base_t),
                       CP_EVAL_PPL="1", CP_EVAL_WINDOWS=str(a.eval_windows), CP_EVAL_OUT=csv, CP_CKPT_RESUME=str(a.ft_run_base + i), CP_B="1")
            o = run_trainer(env, a.nproc, a.port + 1, os.path.join(a.state_dir, f"altpos_eval_{mode}.log"), a.timeout)
            ppl = [ln for ln in o.splitlines() if "PPL" in ln]
            return {"csv": csv, "ppl_line": ppl[-1] if ppl else ""}
        out["modes"].append({"mode": mode, "finetune": steps.run(f"altpos_ft_{mode}", ft), "eval": steps.run(f"altpos_eval_{mode}", ev)})
    out["ran"], out["skipped"] = steps.ran, steps.skipped
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("progressive", "altpos"):
        p = sub.add_parser(name)
        p.add_argument("--state-dir", default=f"{name}_state")
        p.add_argument("--ckpt-dir", default="checkpoints_bluscriptcp")
        p.add_argument("--prefix", default="blumodelcp")
        p.add_argument("--base-run", type=int, default=0)
        p.add_argument("--base-t", type=int, default=4096)
        p.add_argument("--nproc", type=int, default=1)
        p.add_argument("--port", type=int, default=29720)
        p.add_argument("--ft-steps", type=int, default=300)
        p.add_argument("--ft-run-base", type=int, default=100)
        p.add_argument("--ckpt-freq", type=int, default=25)
        p.add_argument("--eval-windows", type=int, default=32)
        p.add_argument("--timeout", type=float, default=None)
        p.add_argument("--wait-idle-mb", type=int, default=0)
        p.add_argument("--env", action="append", default=[], help="KEY=VALUE passed to every trainer run (architecture, data root, mode)")
    p = sub.choices["progressive"]
    p.add_argument("--stages", type=int, nargs="+", default=[16, 32])
    p.add_argument("--head-dim", type=int, default=64)
    p.add_argument("--rope-base", type=float, default=500000.0)
    p.add_argument("--population", type=int, default=48)
    p.add_argument("--generations", type=int, default=30)
    p.add_argument("--pool", type=int, default=1)
    p.add_argument("--search-nproc", type=int, default=1)
    p.add_argument("--search-windows", type=int, default=4)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--ft-batch", type=int, default=1)
    p.add_argument("--rewarmup", type=int, default=100)
    p = sub.choices["altpos"]
    p.add_argument("--modes", nargs="+", default=["cream", "pose", "randpos"])
    p.add_argument("--yarn-scale", type=float, default=4.0)
    a = ap.parse_args(argv)
    if a.wait_idle_mb > 0:
        wait_for_idle_gpus(a.wait_idle_mb)
    res = progressive(a) if a.cmd == "progressive" else altpos(a)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
