"""Experiment tooling on CPU: the GA search against a fake resident evaluator (pool run identical to serial,
dead-worker re-dispatch, resume), sweep failure classification, snapshot tables."""
import os
import subprocess
import sys
import textwrap

import pytest

from context_parallelism_b200.experiments import longrope_search as LS
from context_parallelism_b200.experiments import mem_sweep, mem_table

FAKE = textwrap.dedent('''
    import sys, os
    die_after = int(os.environ.get("FAKE_DIE_AFTER", "0"))
    n = 0
    for line in sys.stdin:
        line = line.strip()
        if line in ("quit", "exit"):
            break
        toks = open(line).read().split()
        vals = [float(t) for t in toks[toks.index("lambda") + 1:]]       # the reference's file layout
        if any(b < a for a, b in zip(vals, vals[1:])):
            print("ERR not monotone", flush=True); continue
        n += 1
        if die_after and n > die_after and not os.path.exists(os.environ["FAKE_FLAG"]):
            open(os.environ["FAKE_FLAG"], "w").close()
            os._exit(3)
        print("PPL %.6f" % (10.0 + sum((v - 1.0 - 0.5 * i) ** 2 for i, v in enumerate(vals))), flush=True)
''')


def _args(workdir, pool, gens=3):
    ns = type("A", (), {})()
    ns.head_dim, ns.scale, ns.orig_len, ns.base, ns.n_hat = 8, 4.0, 64, 10000.0, 0
    ns.population, ns.generations, ns.pool, ns.seed, ns.workdir, ns.fresh = 8, gens, pool, 0, str(workdir), False
    return ns


def test_ga_pool_equals_serial_and_redispatch(tmp_path, monkeypatch):
    fake = tmp_path / "fake_eval.py"
    fake.write_text(FAKE)
    cmd = [sys.executable, str(fake)]
    b1, v1 = LS.search(_args(tmp_path / "serial", 1), cmd)
    b2, v2 = LS.search(_args(tmp_path / "pool", 3), cmd)
    assert b1 == b2 and v1 == v2
    assert v1 < 10.0 + sum((4.0 - 1.0 - 0.5 * i) ** 2 for i in range(4))          # better than the PI seed
    monkeypatch.setenv("FAKE_DIE_AFTER", "2")
    monkeypatch.setenv("FAKE_FLAG", str(tmp_path / "died"))
    b3, v3 = LS.search(_args(tmp_path / "dead", 2), cmd)
    assert (tmp_path / "died").exists() and b3 == b1 and v3 == v1
    # resume: a finished state is picked up and nothing is re-evaluated
    monkeypatch.delenv("FAKE_DIE_AFTER")
    b4, v4 = LS.search(_args(tmp_path / "serial", 1), cmd)
    assert b4 == b1 and os.path.exists(tmp_path / "serial" / "best_factors.txt")


def test_seeds_are_valid_factor_vectors():
    for lam in (LS.seed_pi(32, 8), LS.seed_ntk(32, 8, 64), LS.seed_yarn(32, 8, 64, 5e5, 4096)):
        assert len(lam) == 32 and all(a <= b for a, b in zip(lam, lam[1:])) and lam[0] >= 1.0
    assert LS.repair([0.5, 3.0, 2.0, 100.0], 8.0) == [1.0, 3.0, 3.0, 10.0]


def test_sweep_failure_classification_and_tables(tmp_path):
    assert mem_sweep.is_fail(1, "")
    assert mem_sweep.is_fail(None, "")
    assert mem_sweep.is_fail(0, "RuntimeError: CUDA error: out of memory")
    assert not mem_sweep.is_fail(0, "step 1 | loss 3.2")
    (tmp_path / "a.txt").write_text("# impl=B200 label=1B rotator=fused attn_mode=ring T=8192 B=1 world_size=8\n"
                                    "# CUDA_MEMGETINFO_USED_MB=12345 TOTAL_MB=183359\n# ALLOC_PEAK reserved_mb=11000 active_mb=10500 internal_frag_pct=4.55\n")
    (tmp_path / "limits_1B_ring_ws8.txt").write_text("# label=1B mode=ring rotator=fused ws=8 max_T_ok=262144 first_T_fail=524288\n8192,1,100\n")
    rows = mem_table.collect(str(tmp_path))
    assert rows[0]["T"] == "8192" and rows[0]["CUDA_MEMGETINFO_USED_MB"] == "12345"
    assert "| B200 | 1B | ring | fused | 8 | 8192 | 12345 |" in mem_table.table_md(rows)
    assert "262144 | 524288" in mem_table.limits_md(str(tmp_path))


def test_mem_sweep_runs_trainer_on_cpu(tmp_path):
    env = ["CP_N_EMBD=32", "CP_N_LAYER=1", "CP_N_HEAD=4", "CP_N_KVHEAD=2", "CP_HEAD_DIM=8", "CP_FFN=64", "CP_VOCAB=97"]
    argv = ["--trainer", "llama", "--nproc", "1", "--mode", "ring", "--rotator", "p2p", "--label", "tiny", "--t-start", "32", "--t-max", "64",
            "--out", str(tmp_path), "--timeout", "300"] + sum((["--env", e] for e in env), [])
    ap_res = mem_sweep.sweep(_parse(argv))
    assert ap_res["max_T_ok"] == 64 and ap_res["first_T_fail"] == 0
    assert len([r for r in mem_table.collect(str(tmp_path))]) == 2


def _parse(argv):
    import argparse
    ap = argparse.ArgumentParser()
    for name, kw in (("--trainer", {}), ("--nproc", {"type": int}), ("--mode", {}), ("--rotator", {}), ("--label", {}), ("--batch", {"type": int, "default": 1}),
                     ("--t-start", {"type": int}), ("--t-max", {"type": int}), ("--bisect", {"type": int, "default": 0}), ("--steps", {"type": int, "default": 2}),
                     ("--timeout", {"type": float}), ("--port", {"type": int, "default": 29651}), ("--out", {}), ("--env", {"action": "append", "default": []})):
        ap.add_argument(name, **kw)
    return ap.parse_args(argv)


def test_progressive_pipeline_resumes_from_done_markers(tmp_path):
    """Search -> fine-tune -> eval for one extension stage on a tiny CPU model; a second run of the same command skips
    every finished sub-step; the GPU-idle poll returns once usage drops."""
    from context_parallelism_b200.experiments import pipeline as P
    arch = ["CP_N_EMBD=32", "CP_N_LAYER=1", "CP_N_HEAD=4", "CP_N_KVHEAD=2", "CP_HEAD_DIM=8", "CP_FFN=64", "CP_VOCAB=97", "CP_SYNTHETIC=1",
            "CP_ATTN_MODE=ring", "CP_ROTATOR=p2p"]
    ck = tmp_path / "ck"
    env = dict(os.environ, **dict(e.split("=") for e in arch), CP_CKPT="1", CP_CKPT_DIR=str(ck), CP_LOG_DIR=str(tmp_path), CP_T="32", CP_B="1",
               CP_GLOBAL_BATCH="32", CP_MAX_STEPS="2", CP_CKPT_FREQ="2", CP_VAL_FREQ="0")
    r = subprocess.run([sys.executable, "-m", "context_parallelism_b200.trainers.llama_cp"], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    argv = ["progressive", "--state-dir", str(tmp_path / "state"), "--ckpt-dir", str(ck), "--base-t", "32", "--stages", "2", "--head-dim", "8",
            "--population", "4", "--generations", "2", "--search-windows", "1", "--eval-windows", "1", "--ft-steps", "2", "--ckpt-freq", "2",
            "--rewarmup", "1", "--timeout", "300", "--port", "29790"] + sum((["--env", e] for e in arch), [])
    saved = dict(os.environ)
    try:
        ap_args = _pipeline_args(argv)
        res = P.progressive(ap_args)
        assert res["ran"] == ["search_s2", "finetune_s2", "eval_s2"] and res["skipped"] == []
        assert (tmp_path / "state" / "eval_s2.done").exists() and (tmp_path / "state" / "ppl_prog_s2.csv").exists()
        assert (ck / "blumodelcp_run100_step_4.ckpt").exists()                  # base step 2 + 2 fine-tune steps, in the stage's own run
        res2 = P.progressive(_pipeline_args(argv))
        assert res2["ran"] == [] and res2["skipped"] == ["search_s2", "finetune_s2", "eval_s2"]
    finally:
        os.environ.clear()
        os.environ.update(saved)
    used = iter([[9000, 10], [100, 10]])
    assert P.wait_for_idle_gpus(500, poll_s=0.01, query=lambda: next(used))
    assert not P.wait_for_idle_gpus(5, poll_s=0.01, max_wait_s=0.05, query=lambda: [100])


def _pipeline_args(argv):
    from context_parallelism_b200.experiments import pipeline as P
    import argparse
    holder = {}
    real = argparse.ArgumentParser.parse_args

    def grab(self, args=None, namespace=None):
        holder["a"] = real(self, args, namespace)
        raise SystemExit(0)
    argparse.ArgumentParser.parse_args = grab
    try:
        try:
            P.main(argv)
        except SystemExit:
            pass
    finally:
        argparse.ArgumentParser.parse_args = real
    return holder["a"]
