"""Context-parallel training on CPU ranks (gloo): ring (HeadTail, three rotators), Ulysses (MHA / GQA / KV
replication), hybrid and DP×CP all reproduce the unsharded run."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
_PORT = [29600]


def run_worker(nproc, *args, device="cpu", timeout=600):
    _PORT[0] += 1
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_PORT[0] + (os.getpid() % 200)),
           os.path.join(HERE, "mp_worker.py"), "--device", device, *map(str, args)]
    env = dict(os.environ, OMP_NUM_THREADS="1", NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    line = [l for l in r.stdout.splitlines() if l.startswith("{")]
    log_dir = os.environ.get("CP_TEST_LOG_DIR")            # keep the complete output of a failing worker for later reading
    if log_dir and (r.returncode != 0 or not line or not json.loads(line[-1]).get("ok")):
        os.makedirs(log_dir, exist_ok=True)
        with open(os.path.join(log_dir, f"worker_fail_{_PORT[0]}.log"), "w") as f:
            f.write(" ".join(cmd) + "\n--- stdout\n" + r.stdout + "\n--- stderr\n" + r.stderr)
    assert r.returncode == 0 and line, f"worker failed rc={r.returncode}\nstdout:\n{r.stdout[-3000:]}\nstderr:\n{r.stderr[-3000:]}"
    res = json.loads(line[-1])
    assert res["ok"], res
    return res


@pytest.mark.parametrize("rotator", ["p2p", "alltoall", "allgather"])
def test_ring_rotators_ws2(rotator):
    run_worker(2, "--mode", "ring", "--rotator", rotator, "--tol", 1e-4)


@pytest.mark.parametrize("extra", [["--lb", 0], ["--recompute", "full"], ["--recompute-k", 1]])
def test_ring_ws2_variants(extra):
    """Contiguous (not load-balanced) shards, full activation recompute (the ring re-runs inside backward), and
    K/V re-rotation in backward instead of saved blocks (``CP_RECOMPUTE_K``)."""
    run_worker(2, "--mode", "ring", "--rotator", "p2p", "--tol", 1e-4, *extra)


@pytest.mark.parametrize("mode,rot,kv", [("ring", "p2p", 2), ("ring", "allgather", 4), ("ulysses", "alltoall", 2), ("ulysses", "alltoall", 1)])
def test_forward_cp_shard_and_unshard_ws2(mode, rot, kv):
    """forward_cp(unshard, pre_sharded) in all four combinations, forward and gradients, against the dense oracle."""
    res = run_worker(2, "--mode", mode, "--rotator", rot, "--kv", kv, "--fcp-test", 1)
    assert res["fcp_test"] and res["worst_cos"] > 0.99999


def test_ring_ws4_gpt2():
    run_worker(4, "--mode", "ring", "--rotator", "p2p", "--family", "gpt2", "--tol", 1e-4)


@pytest.mark.parametrize("kv", [4, 2, 1])
def test_ulysses_ws2_gqa(kv):
    run_worker(2, "--mode", "ulysses", "--rotator", "alltoall", "--kv", kv, "--tol", 1e-4)


def test_ulysses_ws4_kv_replication():
    run_worker(4, "--mode", "ulysses", "--rotator", "alltoall", "--kv", 2, "--tol", 1e-4)


def test_hybrid_ws4():
    run_worker(4, "--mode", "hybrid", "--ulysses", 2, "--rotator", "p2p", "--kv", 2, "--tol", 1e-4)


def test_dp_times_cp_ws4():
    run_worker(4, "--mode", "ring", "--cp", 2, "--rotator", "p2p", "--tol", 1e-4, "--recompute", "selective")
