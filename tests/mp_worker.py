"""Multi-process parity worker (launched by torch.distributed.run from the tests).

Every rank trains the same tiny model for a few steps under context parallelism and compares the loss
trajectory and the final weights with an unsharded single-process run of the same batch: the CP-invariance
check of the reference (Tests/bluscriptcp/cp_parity.sh:46-55; Tests/cp_rope_standin_parity.cpp:117-153).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--family", default="llama")
    ap.add_argument("--mode", default="ring")
    ap.add_argument("--rotator", default="p2p")
    ap.add_argument("--cp", type=int, default=0)
    ap.add_argument("--ulysses", type=int, default=1)
    ap.add_argument("--T", type=int, default=256)
    ap.add_argument("--B", type=int, default=2)
    ap.add_argument("--kv", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--tol", type=float, default=2e-3)
    ap.add_argument("--recompute", default="none")
    ap.add_argument("--ring-outer", type=int, default=0)
    a = ap.parse_args()

    from context_parallelism_b200.config import Config
    from context_parallelism_b200.engine import TrainEngine
    from context_parallelism_b200.parallel.mesh import init_distributed
    rank, world, local = init_distributed("nccl" if a.device == "cuda" else "gloo", timeout_s=120)
    dev = torch.device("cuda", local) if a.device == "cuda" else torch.device("cpu")
    cp = a.cp or world
    head_dim = 64 if a.device == "cuda" else 16
    kw = dict(n_embd=4 * head_dim, n_layer=2, n_head=4, n_kv_head=a.kv if a.family == "llama" else 4, head_dim=head_dim,
              ffn_hidden=8 * head_dim if a.family == "llama" else 16 * head_dim, vocab_size=509, T=a.T, B=a.B, max_steps=50,
              warmup_steps=1, checkpointing=False, recompute=a.recompute, dtype="bf16" if a.device == "cuda" else "fp32",
              weight_tying=(a.family == "gpt2"))
    cfg = Config.from_env(a.family, world, env={}).replace(cp_size=cp, attn_mode=a.mode, rotator=a.rotator,
                                                           ulysses_size=a.ulysses, ring_outer=bool(a.ring_outer), **kw)
    eng = TrainEngine(cfg, dev)
    ref = TrainEngine(cfg.replace(world_size=1, cp_size=1, ulysses_size=1, attn_mode="ring"), dev, standalone=True)
    dp = world // cp
    dp_rank = eng.cp.dp_rank
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, cfg.vocab_size, (a.B * dp, a.T + 1), generator=g).to(dev)
    mine = tok[dp_rank * a.B:(dp_rank + 1) * a.B]
    ok, msgs = True, []
    for s in range(a.steps):
        l = eng.global_loss(eng.train_step(mine[:, :-1], mine[:, 1:]))
        # the unsharded run sees the whole global batch (grad accumulation over the dp slices)
        lr = 0.0
        for d in range(dp):
            sl = tok[d * a.B:(d + 1) * a.B]
            lr += float(ref.forward_backward(sl[:, :-1], sl[:, 1:], accum=dp, last=True)) / dp
        ref.optimizer_step()
        rel = abs(float(l) - lr) / abs(lr)
        msgs.append((s, float(l), lr))
        if not rel < a.tol:
            ok = False
    eng.check_kernels()
    wa, wb = eng.flat.full_master(), ref.flat.full_master()
    cos = float((wa.double() @ wb.double()) / (wa.double().norm() * wb.double().norm()))
    dmax = float((wa - wb).abs().max())
    if cos < (0.99999 if a.tol < 1e-3 else 0.999):
        ok = False
    res = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(res, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"ok": bool(res.item() > 0.5), "losses": msgs, "weight_cos": cos, "weight_maxdiff": dmax,
                          "mode": a.mode, "rotator": a.rotator, "world": world}))
    eng.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if res.item() > 0.5 else 1)


if __name__ == "__main__":
    main()
