"""Evolutionary search of LongRoPE rescale factors against a resident evaluator.

The evaluator is the Llama trainer started with ``CP_LONGROPE_SEARCH=1``: it keeps the model resident,
reads one factor-file path per line on stdin and answers ``PPL <value>`` (or ``ERR ...``) on stdout
(``context_parallelism_b200.trainers.llama_cp``).  This driver mirrors the reference's search tool
(Tests/bluscriptcp/longrope_search.py): population 64, per-dimension resampling with probability 0.3,
monotone non-decreasing repair by running maximum, PI / NTK / YaRN seeds (:109-127), a pool of evaluator
workers with re-dispatch of a dead worker's candidate (:261-281), and a resumable memo + state written with
atomic renames (:313-347).  A pool run is bit-identical to a serial run because candidates are evaluated
by content and results are consumed in candidate order.

    python -m context_parallelism_b200.experiments.longrope_search --head-dim 64 --scale 8 --orig-len 4096 \
        --generations 20 --pool 2 --workdir search_out -- torchrun --nproc-per-node 2 -m context_parallelism_b200.trainers.llama_cp
"""
from __future__ import annotations

import argparse
import json
import math
import os
import random
import subprocess
import sys
import threading
from typing import Dict, List, Optional, Sequence, Tuple


# ----------------------------------------------------------------------------- candidates
def repair(lam: Sequence[float], scale: float) -> List[float]:
    """Clamp to [1, scale·1.25] and make non-decreasing with a running maximum."""
    out, run = [], 1.0
    for v in lam:
        run = max(run, min(max(float(v), 1.0), scale * 1.25))
        out.append(round(run, 6))
    return out


def seed_pi(half: int, scale: float) -> List[float]:
    return [float(scale)] * half


def seed_ntk(half: int, scale: float, head_dim: int) -> List[float]:
    # NTK-aware base change: base' = base * s^(d/(d-2))  =>  lambda_i = s^(2i/(d-2))
    return repair([scale ** (2.0 * i / max(1, head_dim - 2)) for i in range(half)], scale)


def seed_yarn(half: int, scale: float, head_dim: int, base: float, orig_len: int, beta_fast=32.0, beta_slow=1.0) -> List[float]:
    def dim_of(rot):
        return head_dim * math.log(orig_len / (rot * 2 * math.pi)) / (2 * math.log(base))
    lo, hi = max(math.floor(dim_of(beta_fast)), 0), min(math.ceil(dim_of(beta_slow)), half - 1)
    out = []
    for i in range(half):
        ramp = min(1.0, max(0.0, (i - lo) / max(1e-3, hi - lo)))
        out.append(1.0 / ((1.0 / scale) * ramp + (1.0 - ramp)))
    return repair(out, scale)


def mutate(parent: Sequence[float], rng: random.Random, scale: float, p: float = 0.3) -> List[float]:
    child = [rng.uniform(1.0, scale * 1.25) if rng.random() < p else v for v in parent]
    return repair(child, scale)


def crossover(a: Sequence[float], b: Sequence[float], rng: random.Random, scale: float) -> List[float]:
    return repair([x if rng.random() < 0.5 else y for x, y in zip(a, b)], scale)


def key_of(lam: Sequence[float], n_hat: int) -> str:
    return f"{n_hat}|" + ",".join(f"{v:.6f}" for v in lam)


def write_factors(path: str, lam: Sequence[float], n_hat: int, s: float, search_len: int) -> None:
    """Candidate file in the layout both trainers read (bluscriptCP.cpp:538-572)."""
    from ..ops.rope import write_longrope_factors
    write_longrope_factors(path, lam, n_hat, s, search_len)


# ----------------------------------------------------------------------------- evaluator workers
class Worker:
    def __init__(self, cmd: List[str], env: Dict[str, str], idx: int):
        self.cmd, self.env, self.idx, self.proc = cmd, env, idx, None
        self.start()

    def start(self) -> None:
        self.proc = subprocess.Popen(self.cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=self.env, bufsize=1)

    def alive(self) -> bool:
        return self.proc is not None and self.proc.poll() is None

    def evaluate(self, path: str) -> Optional[float]:
        """PPL for the factor file; None if the worker died (the caller re-dispatches); inf for a rejected file."""
        try:
            self.proc.stdin.write(path + "\n")
            self.proc.stdin.flush()
            while True:
                line = self.proc.stdout.readline()
                if not line:
                    return None
                if line.startswith("PPL"):
                    return float(line.split()[1])
                if line.startswith("ERR"):
                    return float("inf")
        except (BrokenPipeError, OSError, ValueError):
            return None

    def close(self) -> None:
        if self.alive():
            try:
                self.proc.stdin.write("quit\n")
                self.proc.stdin.flush()
                self.proc.wait(timeout=60)
            except Exception:
                self.proc.kill()


class Evaluator:
    def __init__(self, cmd: List[str], pool: int, workdir: str, n_hat: int, scale: float, search_len: int, extra_env: Dict[str, str]):
        self.workdir, self.n_hat, self.scale, self.search_len = workdir, n_hat, scale, search_len
        env = dict(os.environ, CP_LONGROPE_SEARCH="1", **extra_env)
        self.workers = [Worker(cmd, dict(env, MASTER_PORT=str(29700 + i)), i) for i in range(max(1, pool))]
        self.memo_path = os.path.join(workdir, "memo.json")
        self.memo: Dict[str, float] = json.load(open(self.memo_path)) if os.path.exists(self.memo_path) else {}
        self.redispatched = 0
        self._lock = threading.Lock()

    def _save_memo(self) -> None:
        tmp = self.memo_path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.memo, f)
        os.replace(tmp, self.memo_path)

    def evaluate_all(self, cands: List[List[float]]) -> List[float]:
        todo = []
        for c in cands:
            k = key_of(c, self.n_hat)
            if k not in self.memo and k not in [t[0] for t in todo]:
                todo.append((k, c))
        queue = list(enumerate(todo))
        deaths: Dict[str, int] = {}

        def run(worker: Worker) -> None:
            while True:
                with self._lock:
                    if not queue:
                        return
                    i, (k, c) = queue.pop(0)
                path = os.path.join(self.workdir, f"cand_w{worker.idx}.txt")
                write_factors(path, c, self.n_hat, self.scale, self.search_len)
                v = worker.evaluate(path)
                if v is None:                       # dead worker: put the candidate back, try to restart, else leave
                    with self._lock:
                        queue.insert(0, (i, (k, c)))
                        self.redispatched += 1
                        deaths[k] = deaths.get(k, 0) + 1
                        if deaths[k] > 3:           # the same candidate keeps killing its evaluator: give up, do not spin
                            return
                    try:
                        worker.start()
                    except Exception:
                        return
                    if not worker.alive():
                        return
                    continue
                with self._lock:
                    self.memo[k] = v
        threads = [threading.Thread(target=run, args=(w,)) for w in self.workers]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if queue:
            raise RuntimeError("every evaluator worker died")
        self._save_memo()
        return [self.memo[key_of(c, self.n_hat)] for c in cands]

    def close(self) -> None:
        for w in self.workers:
            w.close()


# ----------------------------------------------------------------------------- search
def search(args, cmd: List[str]) -> Tuple[List[float], float]:
    os.makedirs(args.workdir, exist_ok=True)
    half = args.head_dim // 2
    search_len = int(args.orig_len * args.scale)
    ev = Evaluator(cmd, args.pool, args.workdir, args.n_hat, args.scale, search_len, {})
    state_path = os.path.join(args.workdir, "state.json")
    rng = random.Random(args.seed)
    if os.path.exists(state_path) and not args.fresh:
        st = json.load(open(state_path))
        pop, gen0, best, best_v = st["pop"], st["gen"], st["best"], st["best_v"]
        rng.setstate(tuple(tuple(x) if isinstance(x, list) else x for x in st["rng"]))
    else:
        seeds = [seed_pi(half, args.scale), seed_ntk(half, args.scale, args.head_dim),
                 seed_yarn(half, args.scale, args.head_dim, args.base, args.orig_len)]
        pop = list(seeds)
        while len(pop) < args.population:
            pop.append(mutate(rng.choice(seeds), rng, args.scale))
        gen0, best, best_v = 0, None, float("inf")
    try:
        for gen in range(gen0, args.generations):
            scores = ev.evaluate_all(pop)
            order = sorted(range(len(pop)), key=lambda i: (scores[i], i))
            if scores[order[0]] < best_v:
                best, best_v = pop[order[0]], scores[order[0]]
            print(f"gen {gen} BEST {best_v:.6f} mean {sum(s for s in scores if math.isfinite(s)) / max(1, sum(math.isfinite(s) for s in scores)):.6f}", flush=True)
            parents = [pop[i] for i in order[: max(2, args.population // 4)]]
            nxt = [parents[0]]
            while len(nxt) < args.population:
                nxt.append(mutate(rng.choice(parents), rng, args.scale) if rng.random() < 0.5
                           else crossover(rng.choice(parents), rng.choice(parents), rng, args.scale))
            pop = nxt
            tmp = state_path + ".tmp"
            with open(tmp, "w") as f:
                json.dump({"pop": pop, "gen": gen + 1, "best": best, "best_v": best_v, "rng": rng.getstate()}, f)
            os.replace(tmp, state_path)
    finally:
        ev.close()
    write_factors(os.path.join(args.workdir, "best_factors.txt"), best, args.n_hat, args.scale, search_len)
    print(f"BEST {best_v:.6f} redispatched {ev.redispatched}", flush=True)
    return best, best_v


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--scale", type=float, default=8.0)
    ap.add_argument("--orig-len", type=int, default=4096)
    ap.add_argument("--base", type=float, default=500000.0)
    ap.add_argument("--n-hat", type=int, default=0)
    ap.add_argument("--population", type=int, default=64)
    ap.add_argument("--generations", type=int, default=10)
    ap.add_argument("--pool", type=int, default=1)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--workdir", default="longrope_search_out")
    ap.add_argument("--fresh", action="store_true")
    ap.add_argument("cmd", nargs=argparse.REMAINDER, help="-- evaluator command")
    args = ap.parse_args(argv)
    cmd = args.cmd[1:] if args.cmd and args.cmd[0] == "--" else args.cmd
    if not cmd:
        cmd = [sys.executable, "-m", "context_parallelism_b200.trainers.llama_cp"]
    search(args, cmd)


if __name__ == "__main__":
    main()
