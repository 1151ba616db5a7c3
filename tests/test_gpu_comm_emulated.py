"""The peer-memory communication kernels and the fused context-parallel paths on ONE GPU.

N arenas on one device stand in for the arenas of N ranks (``parallel.fused.EmulatedHeap``): the peer table of every
emulated rank holds local addresses, so each kernel runs with exactly the index arithmetic, tables and epilogues it
uses across NVLink.  Every fused operation is a sequence of phases separated by cross-rank barriers; here each phase
runs for every emulated rank in turn on one stream (kernels never wait for one another), and the results are compared
with a plain PyTorch restatement on the gathered tensors: the op-level parity the reference checks on 2 and 4 GPUs
(Tests/cp_rope_standin_parity.cpp:117-153, Tests/cp_ulysses_parity.cpp:650-686), including GQA with
1 < kv_heads < q_heads, the case the reference's fused kernel gets wrong (cp_ulysses_parity.cpp:345-356).
"""
import pytest
import torch

from util import assert_close

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda", 0)


def status_ok():
    from context_parallelism_b200 import _native as nv
    torch.cuda.synchronize()
    nv.status_for(dev()).check()


def make_comms(n, mode, n_layer=1, heap_mb=96, **cfg_kw):
    from context_parallelism_b200.config import Config
    from context_parallelism_b200.parallel.fused import EmulatedHeap, FusedComm
    cfg = Config.from_env("llama", 1, env={}).replace(world_size=n, cp_size=n, attn_mode=mode, n_layer=n_layer, **cfg_kw)
    heaps = EmulatedHeap(n, heap_mb << 20, dev())
    grp = (list(range(n)), None)
    out = []
    for r in range(n):
        out.append(FusedComm(cfg, dev(), heaps.for_rank(r), r, n,
                             ring=(grp[0], r) if mode == "ring" else None, uly=(grp[0], r) if mode == "ulysses" else None))
    return cfg, out


def dense_reference(q, k, v, do, scale):
    """fp32 oracle on the full sequence: output, LSE and the three gradients."""
    from context_parallelism_b200.ops import reference as ref
    qf, kf, vf = q.float(), k.float(), v.float()
    o, lse = ref.attention_dense(qf, kf, vf, scale, None, None, True)
    dq, dk, dv = ref.attention_dense_bwd(qf, kf, vf, o, lse, do.float(), scale, None, None, True)
    return o, lse, dq, dk, dv


# ----------------------------------------------------------------------------------------------------- ring
@pytest.mark.parametrize("n,hq,hkv,dkv_mode,lb,D", [(2, 4, 2, "route", True, 64), (4, 4, 2, "route", True, 64), (4, 4, 1, "pull", True, 64),
                                                    (2, 2, 2, "pull", True, 64), (4, 4, 2, "route", False, 64), (2, 4, 4, "pull", False, 64),
                                                    (2, 4, 2, "route", True, 128), (4, 2, 1, "pull", True, 128)])
def test_fused_ring_emulated(n, hq, hkv, dkv_mode, lb, D):
    from context_parallelism_b200.parallel import fused as F
    from context_parallelism_b200.parallel import shard
    torch.manual_seed(n * 10 + hq)
    B, T = 2, 256 * n
    Tl = T // n
    scale = D ** -0.5
    cfg, fcs = make_comms(n, "ring", dkv_mode=dkv_mode, load_balance_ring=lb)
    q = torch.randn(B, T, hq, D, device=dev()).bfloat16()
    k = torch.randn(B, T, hkv, D, device=dev()).bfloat16()
    v = torch.randn(B, T, hkv, D, device=dev()).bfloat16()
    do = torch.randn(B, T, hq, D, device=dev()).bfloat16()
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = dense_reference(q, k, v, do, scale)
    pos = [shard.local_positions(T, n, r, lb).to(dev()) for r in range(n)]
    loc = lambda t, r: t.index_select(1, pos[r]).contiguous()        # noqa: E731
    # forward: publish everywhere, then one attention launch per rank (copy CTAs + compute CTAs)
    st = [F.ring_fwd_publish(fcs[r], loc(k, r), loc(v, r)) for r in range(n)]
    outs = [F.ring_fwd_compute(fcs[r], st[r][0], st[r][1], loc(q, r), pos[r].int(), scale) for r in range(n)]
    status_ok()
    for r in range(n):
        o, lse = outs[r]
        assert_close(o.float(), o_ref.index_select(1, pos[r]), cos=0.9995, rel=3e-2, name=f"ring out rank {r}")
        assert_close(lse, lse_ref.index_select(2, pos[r]), cos=0.99999, rel=1e-2, name=f"ring lse rank {r}")
    # the settled recomputation of CP_SELFCHECK is bit-identical to the overlapped one
    o2, lse2 = F.ring_fwd_settled(fcs[0], st[0][0], loc(q, 0), pos[0].int(), scale)
    torch.cuda.synchronize()
    assert torch.equal(o2, outs[0][0]) and torch.equal(lse2, outs[0][1])
    # sent-versus-received checksums of every chunk (CP_DUMP_KV_CHUNKS)
    for r in range(n):
        sent, received, owners = F.ring_kv_checksums(fcs[r], st[r][0], st[r][1])
        for c, (owner, half) in enumerate(owners):
            s_owner, _, _ = F.ring_kv_checksums(fcs[owner], st[owner][0], st[owner][1])
            assert torch.equal(s_owner[half], received[c]), f"rank {r} chunk {c}"
    # backward: zero, compute (routed red.add or local contributions), finish
    for r in range(n):
        F.ring_bwd_prepare(fcs[r], st[r][0])
    dqs = [F.ring_bwd_compute(fcs[r], st[r][0], st[r][1], loc(q, r), outs[r][0], outs[r][1], loc(do, r), pos[r].int(), scale)
           for r in range(n)]
    dkvs = [F.ring_bwd_finish(fcs[r], st[r][0]) for r in range(n)]
    status_ok()
    for r in range(n):
        assert_close(dqs[r].float(), dq_ref.index_select(1, pos[r]), cos=0.998, rel=5e-2, name=f"ring dq rank {r}")
        assert_close(dkvs[r][0].float(), dk_ref.index_select(1, pos[r]), cos=0.998, rel=5e-2, name=f"ring dk rank {r}")
        assert_close(dkvs[r][1].float(), dv_ref.index_select(1, pos[r]), cos=0.998, rel=5e-2, name=f"ring dv rank {r}")


def test_fused_ring_pull_mode_is_deterministic():
    """Two backward passes over the same inputs give bit-identical dK/dV in pull mode (fixed summation order)."""
    from context_parallelism_b200.parallel import fused as F
    from context_parallelism_b200.parallel import shard
    torch.manual_seed(5)
    n, B, T, hq, hkv, D = 4, 1, 1024, 4, 2, 64
    scale = D ** -0.5
    cfg, fcs = make_comms(n, "ring", dkv_mode="pull")
    q, k, v, do = (torch.randn(B, T, h, D, device=dev()).bfloat16() for h in (hq, hkv, hkv, hq))
    pos = [shard.local_positions(T, n, r, True).to(dev()) for r in range(n)]
    loc = lambda t, r: t.index_select(1, pos[r]).contiguous()        # noqa: E731
    st = [F.ring_fwd_publish(fcs[r], loc(k, r), loc(v, r)) for r in range(n)]
    outs = [F.ring_fwd_compute(fcs[r], st[r][0], st[r][1], loc(q, r), pos[r].int(), scale) for r in range(n)]
    runs = []
    for _ in range(2):
        for r in range(n):
            F.ring_bwd_prepare(fcs[r], st[r][0])
        for r in range(n):
            F.ring_bwd_compute(fcs[r], st[r][0], st[r][1], loc(q, r), outs[r][0], outs[r][1], loc(do, r), pos[r].int(), scale)
        runs.append([F.ring_bwd_finish(fcs[r], st[r][0]).clone() for r in range(n)])
    status_ok()
    for r in range(n):
        assert torch.equal(runs[0][r], runs[1][r])


# ----------------------------------------------------------------------------------------------------- ulysses
@pytest.mark.parametrize("n,hq,hkv", [(2, 4, 2), (4, 8, 2), (4, 4, 4), (2, 4, 1), (4, 12, 4)])
def test_fused_ulysses_emulated(n, hq, hkv):
    """Sequence<->head exchange kernels (KV replication and replica sums when kv_heads < ranks), the attention
    epilogue's scatter into the token owners' arenas, and the mirrored backward."""
    from context_parallelism_b200.parallel import fused as F
    torch.manual_seed(n * 100 + hq * 10 + hkv)
    B, T, D = 2, 128 * n, 64
    Tl = T // n
    scale = D ** -0.5
    cfg, fcs = make_comms(n, "ulysses")
    q = torch.randn(B, T, hq, D, device=dev()).bfloat16()
    k = torch.randn(B, T, hkv, D, device=dev()).bfloat16()
    v = torch.randn(B, T, hkv, D, device=dev()).bfloat16()
    do = torch.randn(B, T, hq, D, device=dev()).bfloat16()
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = dense_reference(q, k, v, do, scale)
    loc = lambda t, r: t[:, r * Tl:(r + 1) * Tl].contiguous()        # noqa: E731
    st = [F.uly_fwd_push(fcs[r], loc(q, r), loc(k, r), loc(v, r)) for r in range(n)]
    # the landing buffers hold this rank's heads of the whole sequence
    ub0 = st[0][0]
    qh, kh, vh = ub0.heads(fcs[0], st[0][1])
    assert torch.equal(qh, q[:, :, :ub0.nq])
    kv_head0 = 0                                                      # rank 0 always holds (a replica of) kv head 0
    assert torch.equal(kh[:, :, 0], k[:, :, kv_head0]) and torch.equal(vh[:, :, 0], v[:, :, kv_head0])
    lses = [F.uly_fwd_compute(fcs[r], st[r][0], st[r][1], scale) for r in range(n)]
    status_ok()
    for r in range(n):
        ub, slot = st[r]
        out = ub.o_view(fcs[r], slot)
        assert_close(out.float(), loc(o_ref, r), cos=0.9995, rel=3e-2, name=f"ulysses out rank {r}")
        assert_close(lses[r], lse_ref[:, r * ub.nq:(r + 1) * ub.nq], cos=0.99999, rel=1e-2, name=f"ulysses lse rank {r}")
    for r in range(n):
        F.uly_bwd_push(fcs[r], st[r][0], st[r][1], loc(do, r))
    for r in range(n):
        F.uly_bwd_compute(fcs[r], st[r][0], st[r][1], lses[r], scale)
    grads = [F.uly_bwd_pull(fcs[r], st[r][0]) for r in range(n)]
    status_ok()
    for r in range(n):
        dq, dk, dv = grads[r]
        assert_close(dq.float(), loc(dq_ref, r), cos=0.998, rel=5e-2, name=f"ulysses dq rank {r}")
        assert_close(dk.float(), loc(dk_ref, r), cos=0.998, rel=5e-2, name=f"ulysses dk rank {r}")
        assert_close(dv.float(), loc(dv_ref, r), cos=0.998, rel=5e-2, name=f"ulysses dv rank {r}")


# ----------------------------------------------------------------------------------------------------- gradient transport
def _tiny_params(seed):
    g = torch.Generator().manual_seed(seed)
    shapes = [("w0", (96, 40)), ("w1", (33, 24)), ("w2", (130, 64)), ("b0", (40,)), ("b1", (7,)), ("g", (64,))]
    return [(nm, torch.nn.Parameter(torch.randn(sh, generator=g).to(dev()))) for nm, sh in shapes]


@pytest.mark.parametrize("n", [2, 4, 3])
def test_sharded_optimizer_emulated(n):
    """reduce-scatter (fp32 over 'peers') -> squared-norm exchange -> AdamW on the owned slices -> all-gather, against the
    replicated optimiser fed with the averaged gradient; sizes are odd on purpose (ragged last slices, a bucket that
    straddles the matrix/vector boundary)."""
    from context_parallelism_b200.ops.optim import AdamW, FlatParams
    cfg, fcs = make_comms(n, "ring", heap_mb=16)
    flats = [FlatParams(_tiny_params(3), True, shard=fcs[r], bucket_elems=4000) for r in range(n)]
    for f in flats:
        assert f.sharded and len(f.buckets) >= 3          # several buckets, the last one holds matrices and vectors
    ref_flat = FlatParams(_tiny_params(3), True, shard=None, bucket_elems=4000)
    opts = [AdamW(f, 1e-2, (0.9, 0.95), 1e-8, 0.1) for f in flats]
    ref_opt = AdamW(ref_flat, 1e-2, (0.9, 0.95), 1e-8, 0.1)
    total = ref_flat.total
    for step in range(3):
        grads = [torch.randn(total, device=dev(), generator=torch.Generator(device=dev()).manual_seed(100 * step + r)) for r in range(n)]
        for r in range(n):
            flats[r].grad.copy_(grads[r])
        ref_flat.grad.copy_(torch.stack(grads).sum(0) / n)
        for r in range(n):
            for b in range(len(flats[r].plan.buckets)):
                fcs[r].reduce_scatter_launch(flats[r], b)
        for r in range(n):
            opts[r].step_count += 1
            flats[r].local_sumsq_()
            fcs[r].share_scalar_launch(flats[r].sumsq, flats[r].slots_off)
        for r in range(n):
            fcs[r].sum_slots_launch(flats[r].sumsq, flats[r].slots)
            opts[r].update_shard_(1e-2, 1.0)
        for r in range(n):
            fcs[r].allgather_launch(flats[r])
        ref_norm = ref_opt.step(1e-2, 1.0)
        status_ok()
        for r in range(n):
            assert abs(float(flats[r].sumsq.sqrt()) - float(ref_norm)) < 1e-4 * float(ref_norm)
            # every rank ends with the same compute copies, equal to the replicated optimiser's
            assert torch.equal(flats[r].p16, flats[0].p16) and torch.equal(flats[r].p32, flats[0].p32)
            nd = ref_flat.n_decay
            assert_close(flats[r].p16[:nd].float(), ref_flat.p16.float(), cos=0.999999, rel=1e-2, name="bf16 copy")
            assert_close(flats[r].p32[: total - nd], ref_flat.master[nd:], cos=0.9999999, rel=1e-5, name="fp32 copy")
    # shards reassemble into the replicated masters
    full = torch.zeros(total, device=dev())
    for r in range(n):
        for a, c, sb in flats[r].plan.owned():
            full[a:c] = flats[r].master[sb:sb + c - a]
    assert_close(full, ref_flat.master, cos=0.9999999, rel=1e-5, name="masters")


@pytest.mark.parametrize("n,numel", [(2, 8), (4, 24), (4, 1000), (3, 4099)])
def test_two_shot_allreduce_emulated(n, numel):
    """The replicated-optimiser transport: bf16 staging, owner reduce, gather; odd sizes and sizes below world*8."""
    from context_parallelism_b200 import _native as nv
    cfg, fcs = make_comms(n, "ring", heap_mb=8)
    bufs = [torch.randn(numel, device=dev()) for _ in range(n)]
    want = torch.stack([(b / n).bfloat16().float() for b in bufs]).sum(0)
    offs = [fc.heap.alloc("grad_stage", numel * 2 + 64) for fc in fcs]
    s = nv.stream_ptr(dev())
    for r, fc in enumerate(fcs):
        stage = fc.heap.view(offs[r], (numel,), torch.bfloat16)
        nv.call("cast_f32_bf16", nv.ptr(bufs[r]), nv.ptr(stage), nv.l(numel), nv.f(1.0 / n), s)
    for r, fc in enumerate(fcs):
        g = fc.g_world
        nv.call("allreduce_reduce", nv.ptr(g.peers), nv.l(offs[r]), nv.ptr(bufs[r]), nv.l(numel), nv.i(n), nv.i(r), nv.i(4), s)
    for r, fc in enumerate(fcs):
        g = fc.g_world
        nv.call("allreduce_gather", nv.ptr(g.peers), nv.l(offs[r]), nv.ptr(bufs[r]), nv.l(numel), nv.i(n), nv.i(r), nv.i(4), s)
    status_ok()
    for r in range(n):
        assert torch.equal(bufs[r], bufs[0]), "every rank must hold the same bits (owner keeps the rounded values)"
        assert_close(bufs[r], want, cos=0.9999, rel=2e-2, name="allreduce")


# ----------------------------------------------------------------------------------------------------- barrier
def test_barrier_kernel_flags_and_timeout():
    """(a) With every other rank's epoch already in place the last rank's barrier returns at once and has written its
    epoch into slot [rank] of every rank's flag row.  (b) A flag that nothing sets makes the bounded wait run out after
    about a millisecond: the kernel returns, the status word holds the time-out code and the host raises."""
    import ctypes
    from context_parallelism_b200 import _native as nv
    from context_parallelism_b200.parallel.fused import FLAG_BYTES
    n = 4
    cfg, fcs = make_comms(n, "ring", heap_mb=4)
    fc = fcs[2]
    g = fc.g_world
    rows = [f.heap.view(g.flag_off, (FLAG_BYTES // 4,), torch.int32) for f in fcs]
    epoch = 7
    for r in range(n):
        if r != 2:
            rows[2][r] = epoch                 # the others "arrived": their epochs sit in rank 2's row
    st = nv.status_for(dev())
    st.buf.zero_()
    nv.call("barrier", nv.ptr(g.peers), nv.l(g.flag_off), nv.i(n), nv.i(2), nv.i(epoch), ctypes.c_double(0.5), st.ptr(), nv.stream_ptr(dev()))
    torch.cuda.synchronize()
    st.check("barrier")                        # no time-out
    for r in range(n):
        assert int(rows[r][2]) == epoch
    # (b) epoch 8 never arrives from rank 0: the wait on rank 2's own row gives up
    rows[2][1] = 8
    rows[2][3] = 8
    nv.call("barrier", nv.ptr(g.peers), nv.l(g.flag_off), nv.i(n), nv.i(2), nv.i(8), ctypes.c_double(1e-3), st.ptr(), nv.stream_ptr(dev()))
    torch.cuda.synchronize()                   # the kernel returned by itself
    code, site, block, aux = st.buf.tolist()
    assert code == 2 and site == 2000 and aux == 0, (code, site, block, aux)
    with pytest.raises(nv.NativeError, match="flag wait timed out"):
        st.check("barrier")
    assert st.buf.tolist()[0] == 0             # the word is cleared for the next step
    y = torch.ones(8, device=dev()) * 2        # the context is alive
    assert float(y.sum()) == 16.0
