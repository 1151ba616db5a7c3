"""CP-invariance gate on the trainer binaries: the per-position perplexity CSV of the Llama trainer must be the
same (relative tolerance 1e-3) for CP = 1, ring CP = 2/4 and Ulysses CP = 2, with every transport; and swapping
the RoPE cache must change the result (the cache swap takes effect).  Counterpart of
Tests/bluscriptcp/cp_parity.sh:46-77 and Tests/hybrid_cp_smoke.sh (banner / NaN / step-line checks).

    python -m context_parallelism_b200.experiments.cp_parity --gpus 4 --T 8192
"""
from __future__ import annotations

import argparse
import csv
import os
import subprocess
import sys
import tempfile


def run_eval(nproc: int, mode: str, rotator: str, T: int, out: str, extra: dict, port: int) -> None:
    env = dict(os.environ, CP_EVAL_PPL="1", CP_CKPT="0", CP_EVAL_WINDOWS="2", CP_T=str(T), CP_ATTN_MODE=mode, CP_ROTATOR=rotator,
               CP_EVAL_OUT=out, CP_SYNTHETIC="1", **{k: str(v) for k, v in extra.items()})
    mod = "context_parallelism_b200.trainers.llama_cp"
    cmd = ([sys.executable, "-m", mod] if nproc == 1 else
           [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
            "--master-port", str(port), "-m", mod])
    r = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"eval failed ({mode} x{nproc} {rotator}):\n{r.stdout[-2000:]}\n{r.stderr[-2000:]}")


def read(path: str):
    return [float(r["mean_nll"]) for r in csv.DictReader(open(path))]


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--rtol", type=float, default=1e-3)
    a = ap.parse_args(argv)
    fused = "fused" if a.gpus > 1 else "p2p"
    cases = [("cp1", 1, "ring", "p2p")]
    if a.gpus >= 2:
        cases += [("ring2_fused", 2, "ring", fused), ("ring2_p2p", 2, "ring", "p2p"), ("uly2_fused", 2, "ulysses", fused), ("uly2_a2a", 2, "ulysses", "alltoall")]
    if a.gpus >= 4:
        cases += [("ring4_fused", 4, "ring", fused), ("hybrid2x2", 4, "hybrid", fused)]
    with tempfile.TemporaryDirectory() as d:
        res = {}
        for i, (tag, n, mode, rot) in enumerate(cases):
            out = os.path.join(d, tag + ".csv")
            run_eval(n, mode, rot, a.T, out, {"CP_ULYSSES_SIZE": 2} if mode == "hybrid" else {}, 29720 + i)
            res[tag] = read(out)
        ref = res["cp1"]
        ok = True
        for tag, v in res.items():
            worst = max(abs(x - y) / max(abs(y), 1e-6) for x, y in zip(v, ref))
            good = worst <= a.rtol or tag == "cp1"
            ok &= good
            print(f"{tag:14s} max rel diff vs CP=1: {worst:.3e} {'ok' if good else 'FAIL'}")
        out = os.path.join(d, "yarn.csv")
        run_eval(1, "ring", "p2p", a.T, out, {"YARN_SCALE": 4, "YARN_ORIG_MAXPOS": a.T // 4}, 29750)
        changed = max(abs(x - y) for x, y in zip(read(out), ref)) > 1e-4
        print(f"cache swap takes effect: {'ok' if changed else 'FAIL'}")
        sys.exit(0 if (ok and changed) else 1)


if __name__ == "__main__":
    main()
