"""Throughput / memory comparison harness: the same block stack trained with each attention mode and transport
(fused peer-memory kernels versus the NCCL-only baselines), random tokens, CSV ``step,loss,lr,dt_ms,tok_per_sec,
mem_gpu_mb`` per configuration.  Plays the role of the reference's external-framework comparison
(Scripts/long-context-attention/train_usp_compare.py:84-86), whose third-party USP package is not available
offline; the baseline arm here is this package's own NCCL path.

    torchrun --nproc-per-node 8 -m context_parallelism_b200.experiments.compare_transports --T 131072 --steps 4
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--T", type=int, default=65536)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--out", default="compare_out")
    ap.add_argument("--modes", default="ring:fused,ring:p2p,ring:alltoall,ring:allgather,ulysses:fused,ulysses:alltoall")
    a = ap.parse_args(argv)
    from context_parallelism_b200.config import Config
    from context_parallelism_b200.engine import TrainEngine
    from context_parallelism_b200.parallel.mesh import init_distributed
    from context_parallelism_b200.utils import metrics as M
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    os.makedirs(a.out, exist_ok=True)
    for item in a.modes.split(","):
        mode, rot = item.split(":")
        cfg = Config.from_env("llama", world).replace(T=a.T, B=1, attn_mode=mode, rotator=rot, cp_size=world, checkpointing=False,
                                                      dtype="bf16" if dev.type == "cuda" else "fp32", recompute="selective")
        eng = TrainEngine(cfg, dev)
        log = M.CsvLog(os.path.join(a.out, f"{mode}_{rot}_ws{world}.csv"), "step,loss,lr,dt_ms,tok_per_sec,mem_gpu_mb")
        tok = torch.randint(0, cfg.vocab_size, (1, a.T + 1), generator=torch.Generator().manual_seed(0))
        for s in range(a.steps):
            if dev.type == "cuda":
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            loss = eng.train_step(tok[:, :-1], tok[:, 1:])
            if dev.type == "cuda":
                e1.record(); torch.cuda.synchronize()
                ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
                if world > 1:
                    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                ms = float(ms)
            else:
                ms = 0.0
            log.row(step=s, loss=float(eng.global_loss(loss)), lr=eng.lr_at(s), dt_ms=ms, tok_per_sec=a.T / max(ms, 1e-9) * 1e3, mem_gpu_mb=M.gpu_mem_mb(dev))
        M.log(f"{mode}:{rot} done")
        eng.close()
        del eng
        if dev.type == "cuda":
            torch.cuda.empty_cache()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
