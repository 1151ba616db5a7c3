#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the Llama-style 1B model at T = 131072 under context
parallelism (Ulysses by default, ``--mode ring`` for ring attention), bf16, synthetic uniform-random
tokens, random-init weights.  One sequence of 131072 tokens per optimiser step is split over the N
GPUs of one node (strong scaling); N = 1 runs the same model without communication.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 3 --warmup 3

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, barrier + synchronize on both
sides, max over ranks) over exactly ``--steps`` full optimiser steps with the batch already on the
device; ``e2e`` repeats the measurement through the same public ``TrainEngine.train_step`` call with the
per-step host→device copy of the tokens from pinned memory and a device→host read of the loss inside
the timed region.  With more than one GPU two more fields follow, both measured outside the headline's
timed region: ``ring`` (the same model and sequence under ring attention, the other mode the metric names,
timed the same way) and ``cp_parity`` (one step of a small model under the same parallelism against an
unsharded run of the same batch in the same process: relative loss difference and cosine of the averaged
gradient).  ``--impl reference`` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REF_UNAVAILABLE = ("reference is not installable: its source tree has no setup.py/pyproject.toml, its Makefile needs the "
                   "absent BluTrain tensor library, MPI and mpic++, and its one Python trainer "
                   "(Scripts/Pytorch/gpt2_cp_attnstyle_fp32.py) imports three private torch.distributed ring-attention "
                   "symbols that torch 2.11 no longer has")

MODELS = {
    # BASELINE config 3 / 5: Llama-style 1B
    "llama1b": dict(family="llama", n_embd=2048, n_layer=16, n_head=32, n_kv_head=8, head_dim=64, ffn_hidden=8192,
                    vocab_size=128256, weight_tying=False, rope_theta=5e5),
    # BASELINE config 4: Llama-3-8B shape
    "llama8b": dict(family="llama", n_embd=4096, n_layer=32, n_head=32, n_kv_head=8, head_dim=128, ffn_hidden=14336,
                    vocab_size=128256, weight_tying=False, rope_theta=5e5),
    # BASELINE config 2: GPT-2 124M
    "gpt2_124m": dict(family="gpt2", n_embd=768, n_layer=12, n_head=12, n_kv_head=12, head_dim=64, ffn_hidden=3072,
                      vocab_size=50257, weight_tying=True),
    # profiling-sized: the 1B layer shapes with 2 layers and a small vocabulary (a few GB on the device)
    "small": dict(family="llama", n_embd=2048, n_layer=2, n_head=32, n_kv_head=8, head_dim=64, ffn_hidden=8192,
                  vocab_size=8192, weight_tying=False, rope_theta=5e5),
    "tiny": dict(family="llama", n_embd=512, n_layer=2, n_head=8, n_kv_head=2, head_dim=64, ffn_hidden=1024,
                 vocab_size=8192, weight_tying=False, rope_theta=5e5),
}


class ClockSampler:
    """Samples SM clock and throttle reasons of this process's GPU with nvidia-smi while a region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [s for s in sm if s > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--mode", default=os.environ.get("CP_ATTN_MODE", "ulysses"), choices=["ulysses", "ring", "hybrid"])
    ap.add_argument("--rotator", default=os.environ.get("CP_ROTATOR", "fused"))
    ap.add_argument("--model", default="llama1b", choices=sorted(MODELS))
    ap.add_argument("--T", type=int, default=131072)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ulysses-size", type=int, default=0)
    ap.add_argument("--cp", type=int, default=0, help="context-parallel degree (default: all GPUs); the rest is data parallel")
    ap.add_argument("--yarn-scale", type=float, default=1.0, help="YaRN position-scaling factor (1 = plain RoPE)")
    ap.add_argument("--recompute", default="selective")
    ap.add_argument("--env", nargs="*", default=[], metavar="KEY=VALUE", help="further settings of the CP_* environment surface, "
                                                                              "e.g. CP_SHARE_FWD_ROTATOR=1 CP_DKV_MODE=pull")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the ring timing and the cp_parity step (N > 1)")
    ap.add_argument("--phases", action="store_true", help="after the timed steps run one more step with every kernel launch "
                                                          "bracketed by CUDA events and report device ms per kernel name")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from context_parallelism_b200 import _native as nv
    from context_parallelism_b200.config import Config
    from context_parallelism_b200.engine import TrainEngine
    from context_parallelism_b200.parallel.mesh import init_distributed

    rank, world, local = init_distributed("nccl")
    if world != args.gpus:
        if rank == 0:
            print(f"bench: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run", file=sys.stderr)
        sys.exit(2)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)

    m = dict(MODELS[args.model])
    family = m.pop("family")
    if args.model == "llama8b":
        os.environ.setdefault("CP_INIT_DEVICE", "1")      # 8 B random-init parameters: draw them on the GPU
    cp = args.cp or world
    dp = world // cp
    env = {"CP_SIZE": str(cp)}
    env.update(kv.split("=", 1) for kv in args.env)
    if args.yarn_scale != 1.0:
        env.update(YARN_SCALE=str(args.yarn_scale), YARN_ORIG_MAXPOS=str(args.T / args.yarn_scale))
    tokens_per_step = args.batch * args.T * dp

    def make_cfg(mode, **over):
        usize = args.ulysses_size or (2 if (mode == "hybrid" and cp % 2 == 0) else 1)
        kw = dict(m, T=args.T, B=args.batch, cp_size=cp, attn_mode=mode, rotator=args.rotator, ulysses_size=usize,
                  dtype="bf16", recompute=args.recompute, max_steps=1000, warmup_steps=10,
                  global_batch=args.batch * args.T * dp, checkpointing=False)
        kw.update(over)
        return Config.from_env(family, world, env=env).replace(**kw), usize

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def measure(mode, with_e2e, sample_clocks):
        """Build the engine for ``mode``, warm up, time ``--steps`` optimiser steps on the device (and end to end)."""
        cfg, usize = make_cfg(mode)
        eng = TrainEngine(cfg, dev)
        gen = torch.Generator().manual_seed(1234 + eng.cp.dp_rank)   # all CP ranks of a replica read the same batch; replicas differ
        n_batches = 4
        host = [torch.randint(0, cfg.vocab_size, (args.batch, args.T + 1), generator=gen).pin_memory() for _ in range(n_batches)]
        devb = [h.to(dev) for h in host]

        def step_dev(i):
            b = devb[i % n_batches]
            return eng.train_step(b[:, :-1], b[:, 1:])

        def step_e2e(i):
            h = host[i % n_batches]
            loss = eng.train_step(h[:, :-1], h[:, 1:])      # H2D of the pinned tokens happens inside
            return float(loss)                               # D2H read of the step's loss

        for i in range(args.warmup):
            step_dev(i)
        eng.check_kernels()
        sampler = ClockSampler(local) if sample_clocks else None
        barrier()
        if sampler:
            sampler.start()
        launches0 = nv.LAUNCHES[0]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(args.steps):
            loss = step_dev(args.warmup + i)
        e1.record()
        barrier()
        launches = nv.LAUNCHES[0] - launches0
        ms = max_over_ranks(e0.elapsed_time(e1))
        clocks = sampler.stop() if sampler else None
        eng.check_kernels()
        res = {"cfg": cfg, "usize": usize, "ms": ms, "value": tokens_per_step * args.steps / (ms / 1e3), "clocks": clocks,
               "launches": int(launches), "final_loss": float(eng.global_loss(loss)), "e2e": None,
               "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30, "sharded_optimizer": bool(eng.flat.sharded)}
        if with_e2e:
            step_e2e(0)
            barrier()
            e0.record()
            for i in range(args.steps):
                step_e2e(i + 1)
            e1.record()
            barrier()
            ms2 = max_over_ranks(e0.elapsed_time(e1))
            res["e2e"] = {"value": tokens_per_step * args.steps / (ms2 / 1e3), "unit": "tokens/s",
                          "h2d_bytes_per_step": int(2 * args.batch * args.T * 8), "d2h_bytes_per_step": 4}
        if args.phases:
            # one more step, outside every timed region, with per-launch CUDA events (max over ranks per kernel name)
            barrier()
            nv.profile_start()
            e0.record()
            step_dev(0)
            e1.record()
            prof = nv.profile_stop()
            names = sorted(prof)
            t = torch.tensor([prof[k][1] for k in names] + [e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            if world > 1:
                lists = [None] * world
                dist.all_gather_object(lists, names)
                assert all(l == names for l in lists), "ranks launched different kernels"
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res["phases"] = {"step_ms": float(t[-1]), "kernels": {k: {"calls": prof[k][0], "ms": round(float(t[i]), 3)} for i, k in enumerate(names)}}
        eng.check_kernels()
        eng.close()
        del eng, devb, host
        torch.cuda.empty_cache()
        return res

    def cp_parity(mode):
        """One optimiser-free step of a small model under the job's parallelism against an unsharded run of the same
        global batch on this GPU: relative loss difference and cosine of the averaged gradient (max / min over ranks)."""
        small = dict(MODELS["tiny"])
        small.pop("family")
        Tp = 2048 * cp
        usize = args.ulysses_size or (2 if (mode == "hybrid" and cp % 2 == 0) else 1)
        pcfg = Config.from_env("llama", world, env={"CP_SIZE": str(cp)}).replace(
            **small, T=Tp, B=1, cp_size=cp, attn_mode=mode, rotator=args.rotator, ulysses_size=usize, dtype="bf16",
            recompute="none", max_steps=10, warmup_steps=1, global_batch=Tp * dp, checkpointing=False)
        e = TrainEngine(pcfg, dev)
        r = TrainEngine(pcfg.replace(world_size=1, cp_size=1, ulysses_size=1, attn_mode="ring"), dev, standalone=True)
        g = torch.Generator().manual_seed(4321)
        tok = torch.randint(0, pcfg.vocab_size, (dp, Tp + 1), generator=g).to(dev)
        mine = tok[e.cp.dp_rank:e.cp.dp_rank + 1]
        l_cp = float(e.global_loss(e.forward_backward(mine[:, :-1], mine[:, 1:], 1, True)))
        l_ref = 0.0
        for d in range(dp):
            l_ref += float(r.forward_backward(tok[d:d + 1, :-1], tok[d:d + 1, 1:], accum=dp, last=True)) / dp
        ga, gb = e.flat.full_reduced_grad().double(), r.flat.grad.double()
        cos = float((ga @ gb) / (ga.norm() * gb.norm() + 1e-30))
        t = torch.tensor([abs(l_cp - l_ref) / abs(l_ref), -cos], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e.check_kernels()
        e.close()
        return {"loss_rel": float(t[0]), "grad_cos": float(-t[1]), "model": "tiny", "seq_len": Tp, "mode": mode}

    mode = args.mode
    main_res = measure(mode, not args.no_e2e, True)
    cfg, usize, ms = main_res["cfg"], main_res["usize"], main_res["ms"]
    value, clocks, e2e, launches, final_loss = (main_res[k] for k in ("value", "clocks", "e2e", "launches", "final_loss"))
    ring_res = parity = None
    if world > 1 and not args.no_extras:
        parity = {mode: cp_parity(mode)}
        if mode != "ring" and cp > 1:
            rr = measure("ring", False, False)
            ring_res = {"value": rr["value"], "unit": "tokens/s", "ms_per_step": rr["ms"] / args.steps, "steps": args.steps,
                        "warmup": args.warmup, "final_loss": rr["final_loss"], "parallelism": f"ring{cp}" + (f"xdp{dp}" if dp > 1 else "")}
            parity["ring"] = cp_parity("ring")

    # model FLOPs per step (whole job): dense matmuls 6*P_active*tokens + causal attention 3.5 * 2*T^2*d_attn*L
    p_dense = cfg.n_layer * (cfg.n_embd * (cfg.n_head + 2 * cfg.n_kv_head) * cfg.head_dim + cfg.n_head * cfg.head_dim * cfg.n_embd
                             + (3 if family == "llama" else 2) * cfg.n_embd * cfg.ffn_hidden) + cfg.n_embd * cfg.vocab_size
    attn_flops = 3.5 * 2.0 * args.T * args.T * cfg.n_head * cfg.head_dim * cfg.n_layer * args.batch * dp
    flops = 6.0 * p_dense * tokens_per_step + attn_flops
    if rank == 0:
        par = "single" if world == 1 else (f"{mode}{cp}" if mode != "hybrid" else f"hybrid_r{cp // usize}xu{usize}")
        if dp > 1:
            par += f"xdp{dp}"
        print(json.dumps({
            "metric": f"training tokens/sec/box at T={args.T} ({mode} CP, {args.model})",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
            "config": {"model": args.model, "global_batch": args.batch * dp, "seq_len": args.T, "yarn_scale": args.yarn_scale,
                       "parallelism": par, "rotator": args.rotator if world > 1 else "none",
                       "recompute": args.recompute, "env": sorted(args.env), "l2": "inputs larger than L2 (activations are GBs per layer)",
                       "optimizer_step_in_timed_region": True},
            "model_tflops_per_gpu": flops / (ms / args.steps / 1e3) / world / 1e12,
            "attn_share_of_flops": attn_flops / flops,
            "final_loss": final_loss,
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
            "peak_mem_gb": main_res["peak_mem_gb"], "sharded_optimizer": main_res["sharded_optimizer"],
            "ring": ring_res, "cp_parity": parity, "phases": main_res.get("phases"),
        }))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
