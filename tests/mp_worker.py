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
    ap.add_argument("--pg-test", type=int, default=0)
    ap.add_argument("--fcp-test", type=int, default=0)
    a = ap.parse_args()

    from context_parallelism_b200.config import Config
    from context_parallelism_b200.engine import TrainEngine
    from context_parallelism_b200.parallel.mesh import init_distributed
    rank, world, local = init_distributed("nccl" if a.device == "cuda" else "gloo", timeout_s=120)
    dev = torch.device("cuda", local) if a.device == "cuda" else torch.device("cpu")
    if a.pg_test:
        ok = native_pg_test(rank, world, dev)
        if rank == 0:
            print(json.dumps({"ok": ok, "pg_test": True, "world": world}))
        dist.barrier()
        dist.destroy_process_group()
        sys.exit(0 if ok else 1)
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
    if a.fcp_test:
        res = forward_cp_test(eng, cfg, dev)
        if rank == 0:
            print(json.dumps(res))
        eng.close()
        dist.barrier()
        dist.destroy_process_group()
        sys.exit(0 if res["ok"] else 1)
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


def forward_cp_test(eng, cfg, dev):
    """``forward_cp`` in its four sharding modes against the dense oracle: full-sequence inputs sharded inside
    (``pre_sharded=False``) and/or the output gathered back (``unshard=True``), forward and all three gradients
    (the reference's op-level parity, Tests/cp_ulysses_parity.cpp:650-651, Tests/cp_rope_standin_parity.cpp:117-153)."""
    from context_parallelism_b200.ops import reference as ref
    attn, cp = eng.model.attn, eng.cp
    B, T, Hq, Hkv, D = cfg.B, cfg.T, cfg.n_head, cfg.n_kv_head, cfg.head_dim
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    gen = torch.Generator().manual_seed(5)
    q, k, v, do = (torch.randn(B, T, h, D, generator=gen).to(dev).to(dt) for h in (Hq, Hkv, Hkv, Hq))
    scale = D ** -0.5
    o_ref, lse_ref = ref.attention_dense(q.float(), k.float(), v.float(), scale, None, None, True)
    g_ref = ref.attention_dense_bwd(q.float(), k.float(), v.float(), o_ref, lse_ref, do.float(), scale, None, None, True)
    pos = cp.local_positions(T).to(dev)
    worst = 1.0

    def cos(x, y):
        x, y = x.double().flatten(), y.double().flatten()
        return float((x @ y) / (x.norm() * y.norm() + 1e-30))
    for pre_sharded in (False, True):
        for unshard in (False, True):
            sel = (lambda t: t.index_select(1, pos).contiguous()) if pre_sharded else (lambda t: t.clone())
            qi, ki, vi = (sel(t).requires_grad_() for t in (q, k, v))
            o = attn.forward_cp(qi, ki, vi, unshard=unshard, pre_sharded=pre_sharded)
            o.backward(do if unshard else do.index_select(1, pos))
            want_o = o_ref if unshard else o_ref.index_select(1, pos)
            cs = [cos(o, want_o)]
            for got, want in zip((qi.grad, ki.grad, vi.grad), g_ref):
                cs.append(cos(got, want.index_select(1, pos) if pre_sharded else want))
            worst = min(worst, *cs)
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    lim = 0.995 if dev.type == "cuda" else 0.99999
    return {"ok": bool(t.item() > lim), "worst_cos": float(t.item()), "fcp_test": True, "mode": cfg.attn_mode}


def native_pg_test(rank, world, dev):
    """Every collective of the native NCCL process group against its definition, the ring hop on the dedicated
    communicator, a communicator split, and the work handle's three ways of waiting."""
    from context_parallelism_b200.parallel.process_group import NativeProcessGroup
    from context_parallelism_b200.parallel.work import DONE
    torch.cuda.set_device(dev)
    pg = NativeProcessGroup.create(None, timeout_s=60.0, with_ring=True, device=dev)
    ok = pg.world == world and pg.rank == rank and pg.async_error() == 0
    cur = torch.cuda.current_stream(dev)
    x = torch.full((1000,), float(rank + 1), device=dev)
    w = pg.all_reduce(x, "sum"); w.stream_wait(cur); w.close()
    ok &= bool((x == world * (world + 1) / 2).all())
    y = torch.full((64,), float(rank), device=dev, dtype=torch.bfloat16)
    w = pg.broadcast(y, world - 1)
    ok &= w.wait() == DONE                               # host-side polling wait with the deadline
    w.close()
    ok &= bool((y == world - 1).all())
    g = torch.empty(world * 8, device=dev)
    w = pg.all_gather(torch.full((8,), float(rank), device=dev), g); w.stream_wait(cur); w.close()
    ok &= bool((g.view(world, 8)[:, 0] == torch.arange(world, device=dev)).all())
    rs = torch.empty(4, device=dev)
    w = pg.reduce_scatter(torch.arange(world * 4, device=dev, dtype=torch.float32), rs, "avg"); w.stream_wait(cur); w.close()
    ok &= bool((rs == torch.arange(rank * 4, rank * 4 + 4, device=dev)).all())
    send = (torch.arange(world * 3, device=dev) + 100 * rank).float()
    recv = torch.empty_like(send)
    w = pg.all_to_all(send, recv); w.stream_wait(cur); w.close()
    want = torch.cat([torch.arange(rank * 3, rank * 3 + 3, device=dev).float() + 100 * r for r in range(world)])
    ok &= bool((recv == want).all())
    hop = torch.empty(16, device=dev)
    w = pg.sendrecv(torch.full((16,), float(rank), device=dev), hop, (rank + 1) % world, (rank - 1) % world)
    w.stream_wait(cur)
    ok &= w.query() in (0, 1)
    w.close()
    ok &= bool((hop == (rank - 1) % world).all())
    if world >= 2:
        half = pg.split(rank % 2, rank // 2, (world + 1 - rank % 2) // 2, rank // 2)        # even / odd ranks
        z = torch.ones(4, device=dev)
        w = half.all_reduce(z, "sum"); w.stream_wait(cur); w.close()
        ok &= bool((z == half.world).all())
        torch.cuda.synchronize(dev)
        half.close()
    torch.cuda.synchronize(dev)
    ok &= pg.async_error() == 0
    pg.close()
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item() > 0.5)


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
