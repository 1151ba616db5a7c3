"""Context parallelism on real GPUs (one process per GPU, NCCL + the peer-memory kernels): fused and
NCCL-baseline transports of ring / Ulysses / hybrid reproduce the unsharded run."""
import os

import pytest
import torch

from test_cp_cpu_gloo import run_worker

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0


# Tolerances: the loss of the sharded run follows the unsharded one to about 1e-5 and the weights to cos 0.9999999 in
# practice; 2e-3 / 0.99999 leaves room for bf16 reduction-order effects while a wrong gradient block (one HeadTail
# chunk, one KV replica) moves the loss by far more within three steps.
TOL = 2e-3


@pytest.mark.parametrize("rotator,extra", [("fused", ["--op-parity", 1]), ("fused", ["--dkv-mode", "pull", "--op-parity", 1]),
                                           ("fused", ["--shard-optim", 0]), ("fused", ["--share-slots", 1, "--recompute", "full"]),
                                           ("fused", ["--lb", 0, "--op-parity", 1]), ("p2p", [])])
def test_ring_2gpu(rotator, extra):
    run_worker(2, "--mode", "ring", "--rotator", rotator, "--T", 1024, "--tol", TOL, *extra, device="cuda")


@pytest.mark.parametrize("rotator,kv,extra", [("fused", 2, ["--op-parity", 1]), ("fused", 1, ["--op-parity", 1]),
                                              ("fused", 2, ["--recompute", "full"]), ("alltoall", 2, [])])
def test_ulysses_2gpu(rotator, kv, extra):
    run_worker(2, "--mode", "ulysses", "--rotator", rotator, "--kv", kv, "--T", 1024, "--tol", TOL, *extra, device="cuda")


def test_native_process_group_2gpu():
    """The C++ NCCL process group: collectives, ring hop on the dedicated communicator, split, work handles."""
    res = run_worker(2, "--pg-test", 1, device="cuda")
    assert res["pg_test"]


def test_ring_fused_gpt2_recompute_2gpu():
    run_worker(2, "--mode", "ring", "--rotator", "fused", "--family", "gpt2", "--T", 1024, "--tol", TOL,
               "--recompute", "selective", device="cuda")


@pytest.mark.parametrize("peer_exchange", ["1", "0"])
def test_hybrid_fused_ulysses_exchange_2gpu(monkeypatch, peer_exchange):
    """Hybrid with Ulysses degree 2 and ring degree 1: the peer-memory sequence<->head exchange around the local attention
    (the default) and the NCCL all-to-all on the Ulysses axis."""
    monkeypatch.setenv("CP_FUSED_HYBRID_ULYSSES", peer_exchange)
    run_worker(2, "--mode", "hybrid", "--ulysses", 2, "--rotator", "fused", "--T", 1024, "--tol", TOL, device="cuda")


@pytest.mark.skipif(NGPU < 4, reason="needs 4 GPUs")
def test_hybrid_fused_ulysses_exchange_4gpu(monkeypatch):
    """Ring 2 x Ulysses 2 with the peer-memory exchange on the Ulysses axis as well."""
    monkeypatch.setenv("CP_FUSED_HYBRID_ULYSSES", "1")
    run_worker(4, "--mode", "hybrid", "--ulysses", 2, "--rotator", "fused", "--T", 2048, "--tol", TOL, device="cuda")


@pytest.mark.skipif(NGPU < 4, reason="needs 4 GPUs")
@pytest.mark.parametrize("mode,extra", [("ring", ["--op-parity", 1]), ("ulysses", ["--kv", 2, "--op-parity", 1]),
                                        ("hybrid", ["--ulysses", 2]), ("ring", ["--cp", 2]),
                                        ("ring", ["--dkv-mode", "pull", "--op-parity", 1])])
def test_fused_4gpu(mode, extra):
    run_worker(4, "--mode", mode, "--rotator", "fused", "--T", 2048, "--tol", TOL, *extra, device="cuda")
