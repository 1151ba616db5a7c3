"""Multi-process parity worker (launched by torch.distributed.run from the tests).

Every rank trains the same tiny model for a few steps under context parallelism and compares the loss
trajectory and the final weights with an unsharded single-process run of the same batch: the CP-invariance
check of the reference (Tests/bluscriptcp/cp_parity.sh:46-55; Tests/cp_rope_standin_parity.cpp:117-153).
With ``--op-parity 1`` (CUDA, fused transport) the attention operator itself is checked first: output and
dQ/dK/dV of the fused ring / fused Ulysses on this rank's shard against the dense fp32 oracle on the gathered
tensors, per tensor (cos > 0.999 forward, > 0.995 backward), with 1 < kv_heads < q_heads.  After training the
compute copies of the parameters must be bit-identical on every rank.
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
    ap.add_argument("--op-parity", type=int, default=0)
    ap.add_argument("--dkv-mode", default="route")
    ap.add_argument("--shard-optim", type=int, default=1)
    ap.add_argument("--share-slots", type=int, default=0)
    ap.add_argument("--lb", type=int, default=1)
    ap.add_argument("--recompute-k", type=int, default=0)
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
              weight_tying=(a.family == "gpt2"), dkv_mode=a.dkv_mode, shard_optim=bool(a.shard_optim),
              share_fwd_rotator=bool(a.share_slots), load_balance_ring=bool(a.lb), recompute_k=bool(a.recompute_k))
    cfg = Config.from_env(a.family, world, env={}).replace(cp_size=cp, attn_mode=a.mode, rotator=a.rotator,
                                                           ulysses_size=a.ulysses, ring_outer=bool(a.ring_outer), **kw)
    eng = TrainEngine(cfg, dev)
    ref = TrainEngine(cfg.replace(world_size=1, cp_size=1, ulysses_size=1, attn_mode="ring"), dev, standalone=True)
    dp = world // cp
    dp_rank = eng.cp.dp_rank
    ok, msgs = True, []
    op = None
    if a.op_parity and eng.cp.fused is not None and a.mode in ("ring", "ulysses"):
        op = op_parity(eng, cfg, dev)
        ok = ok and op["ok"]
    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, cfg.vocab_size, (a.B * dp, a.T + 1), generator=g).to(dev)
    mine = tok[dp_rank * a.B:(dp_rank + 1) * a.B]
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
    if cos < (0.99999 if a.tol <= 2e-3 else 0.999):
        ok = False
    # replicas must not drift: every rank holds the same bits of the compute copies
    same = True
    if dev.type == "cuda" and world > 1:
        from context_parallelism_b200.utils.debug import DebugTools
        cs = DebugTools.checksum(eng.flat.p16).to(dev)
        allc = [torch.empty_like(cs) for _ in range(world)]
        dist.all_gather(allc, cs)
        same = all(torch.equal(c, allc[0]) for c in allc)
        ok = ok and same
    res = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(res, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"ok": bool(res.item() > 0.5), "losses": msgs, "weight_cos": cos, "weight_maxdiff": dmax,
                          "mode": a.mode, "rotator": a.rotator, "world": world, "replicas_identical": same, "op_parity": op}))
    eng.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if res.item() > 0.5 else 1)


def op_parity(eng, cfg, dev):
    """Fused attention operator on this rank's shard versus the dense oracle on the whole sequence."""
    from context_parallelism_b200.ops import reference as ref
    fc, cp = eng.cp.fused, eng.cp
    B, T, Hq, Hkv, D = cfg.B, cfg.T, cfg.n_head, cfg.n_kv_head, cfg.head_dim
    scale = D ** -0.5
    gen = torch.Generator().manual_seed(77 + cp.dp_rank)
    full = [torch.randn(B, T, h, D, generator=gen).to(dev).bfloat16() for h in (Hq, Hkv, Hkv, Hq)]
    q, k, v, do = full
    pos = cp.local_positions(T).to(dev)
    ql, kl, vl, dol = (t.index_select(1, pos).contiguous() for t in full)
    ql.requires_grad_(); kl.requires_grad_(); vl.requires_grad_()
    if cfg.attn_mode == "ring":
        out = fc.ring_attention(ql, kl, vl, pos, T, scale)
    else:
        out = fc.ulysses_attention(ql, kl, vl, scale)
    out.backward(dol)
    o_ref, lse_ref = ref.attention_dense(q.float(), k.float(), v.float(), scale, None, None, True)
    dq_ref, dk_ref, dv_ref = ref.attention_dense_bwd(q.float(), k.float(), v.float(), o_ref, lse_ref, do.float(), scale, None, None, True)

    def cos(x, y):
        x, y = x.double().flatten(), y.double().flatten()
        return float((x @ y) / (x.norm() * y.norm() + 1e-30))
    res = {"out": cos(out, o_ref.index_select(1, pos)), "dq": cos(ql.grad, dq_ref.index_select(1, pos)),
           "dk": cos(kl.grad, dk_ref.index_select(1, pos)), "dv": cos(vl.grad, dv_ref.index_select(1, pos))}
    worst = torch.tensor([res["out"] - 0.999, res["dq"] - 0.995, res["dk"] - 0.995, res["dv"] - 0.995], device=dev).min().reshape(1)
    dist.all_reduce(worst, op=dist.ReduceOp.MIN)
    res["ok"] = bool(worst.item() > 0)
    eng.check_kernels()
    return res


if __name__ == "__main__":
    main()
