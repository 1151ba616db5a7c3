"""Host-side logic against the reference's golden values (restated, not copied): RoPE deltas, HeadTail
permutations, CREAM label math, RoPE caches, LR schedules, config parsing, mesh math, merge math."""
import math
import os

import pytest
import torch

from context_parallelism_b200.config import Config
from context_parallelism_b200.ops import reference as R
from context_parallelism_b200.parallel import rope_deltas as RD
from context_parallelism_b200.parallel import shard
from context_parallelism_b200.utils import cream, lr


def test_headtail_perm_examples():
    assert shard.headtail_perm(8, 2).tolist() == [0, 1, 6, 7, 2, 3, 4, 5]
    inv = shard.headtail_inverse_perm(8, 2)
    x = torch.arange(8)
    assert x[shard.headtail_perm(8, 2)][inv].tolist() == list(range(8))
    assert shard.local_positions(8, 2, 0, True).tolist() == [0, 1, 6, 7]
    assert shard.local_positions(8, 2, 1, True).tolist() == [2, 3, 4, 5]
    assert shard.local_positions(16, 4, 1, True).tolist() == [2, 3, 12, 13]
    assert shard.local_positions(8, 2, 1, False).tolist() == [4, 5, 6, 7]
    for r in range(4):
        pos = shard.local_positions(32, 4, r, True).tolist()
        assert [shard.local_to_global_pos(r, i, 8, 4, True) for i in range(8)] == pos
    with pytest.raises(ValueError):
        shard.headtail_perm(10, 4)


def test_hybrid_positions_compose():
    T, Rn, U = 32, 2, 2
    seen = []
    for rr in range(Rn):
        block = shard.local_positions(T, Rn, rr, True)
        for u in range(U):
            p = shard.hybrid_local_positions(T, Rn, rr, U, u)
            assert p.tolist() == block[u * 8:(u + 1) * 8].tolist()
            seen += p.tolist()
    assert sorted(seen) == list(range(T))


@pytest.mark.parametrize("args,want", [
    ((0, 0, 1, 8, False, RD.SubChunk.Full), (0, 0, 0, 0)),
    ((0, 1, 2, 4, False, RD.SubChunk.Full), (0, 0, 4, 4)),
    ((1, 0, 2, 4, False, RD.SubChunk.Full), (4, 4, 4, 4)),
    ((1, 1, 2, 4, False, RD.SubChunk.Full), (4, 4, 0, 0)),
    ((0, 0, 2, 4, True, RD.SubChunk.Full), (0, 4, 0, 4)),
    ((1, 0, 2, 4, True, RD.SubChunk.Full), (2, 2, 2, 2)),
    ((0, 1, 2, 4, True, RD.SubChunk.QTailHalf), (6, 6, 2, 2)),
    ((1, 1, 2, 4, True, RD.SubChunk.KHeadHalf), (2, 2, 0, 0)),
    ((1, 0, 4, 4, True, RD.SubChunk.Full), (2, 10, 2, 10)),
    ((1, 1, 4, 4, True, RD.SubChunk.KHeadHalf), (2, 10, 0, 0)),
    ((1, 2, 4, 4, True, RD.SubChunk.QTailHalf), (12, 12, 6, 6)),
])
def test_rope_delta_table(args, want):
    d = RD.compute_deltas(*args)
    assert (d.q.d0, d.q.d1, d.k.d0, d.k.d1) == want


def test_rope_delta_position_sets():
    d = RD.compute_deltas(0, 0, 2, 4, True, RD.SubChunk.Full)
    assert {RD.rope_global_pos(j, 4, d.q) for j in range(4)} == {0, 1, 6, 7}
    d = RD.compute_deltas(0, 1, 2, 4, True, RD.SubChunk.QTailHalf)
    assert {RD.rope_global_pos(j, 2, d.q) for j in range(2)} == {6, 7}
    assert {RD.rope_global_pos(j, 4, d.k) for j in range(4)} == {2, 3, 4, 5}
    d = RD.compute_deltas(1, 0, 4, 4, True, RD.SubChunk.Full)
    assert {RD.rope_global_pos(j, 4, d.q) for j in range(4)} == {2, 3, 12, 13}
    assert RD.subchunk_for_step(1, 1, True) is RD.SubChunk.KHeadHalf
    assert RD.subchunk_for_step(1, 2, True) is RD.SubChunk.QTailHalf
    assert RD.subchunk_for_step(1, 2, False) is RD.SubChunk.Full


@pytest.mark.parametrize("T,f,b,rf,eid,h", [(256, 8, 0, 8, 700, 44045830), (256, 8, 1, 5, 300, 21283296),
                                            (96, 2, 0, 4, 120, 630640), (300, 4, 1, 6, 900, 38097978)])
def test_cream_labels_golden(T, f, b, rf, eid, h):
    L = cream.cream_labels_from_draws(T, f, b, rf, eid)
    assert len(L) == T and cream.vhash(L) == h
    assert all(L[i] < L[i + 1] for i in range(T - 1)) and L[0] == 0 and L[-1] == f * T - 1


@pytest.mark.parametrize("u,f,want", [(0.01, 2, 2), (0.01, 8, 2), (0.25, 8, 6), (0.5, 2, 3), (0.5, 4, 5), (0.5, 8, 9),
                                      (0.75, 2, 4), (0.75, 4, 7), (0.75, 8, 11), (0.99, 2, 4), (0.99, 4, 8), (0.99, 8, 15)])
def test_cream_rand_factor(u, f, want):
    assert cream.rand_factor_from_u(u, f, 3.0) == want


@pytest.mark.parametrize("T,f,b,rf,lo,hi", [(256, 8, 0, 8, 425, 938), (256, 8, 0, 7, 382, 810), (256, 8, 1, 5, 509, 607),
                                            (96, 2, 0, 4, 94, 159), (300, 4, 1, 7, 950, 1033)])
def test_cream_end_id_range(T, f, b, rf, lo, hi):
    assert cream.end_id_range(T, f, b, rf) == (lo, hi)


def test_cream_generators_structure():
    for seed in range(5):
        for mode in ("cream", "pose", "randpos"):
            L = cream.generate_positions(mode, 256, 8, 3.0, seed)
            assert len(L) == 256 and all(L[i] < L[i + 1] for i in range(255)) and 0 <= L[0] and L[-1] < 8 * 256
    with pytest.raises(ValueError):
        cream.cream_validate(256, 1, 0)
    with pytest.raises(ValueError):
        cream.cream_validate(60, 8, 1)


def test_rope_caches():
    c = R.build_rope_cache(64, 16, 10000.0)
    pos = torch.arange(64, dtype=torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(8, dtype=torch.float32) * 2 / 16))
    assert torch.allclose(c[:, :8], (pos[:, None] * inv).cos(), atol=1e-5)
    assert torch.allclose(c[:, 8:], (pos[:, None] * inv).sin(), atol=1e-5)
    # LongRoPE: lambda = 1 is plain RoPE, lambda = s is position interpolation, n_hat keeps early rows
    assert torch.allclose(R.build_rope_cache_longrope(64, 16, 10000.0, [1.0] * 8, 0), c, atol=1e-6)
    pi = R.build_rope_cache_longrope(64, 16, 10000.0, [4.0] * 8, 0)
    assert torch.allclose(pi[:, :8], (pos[:, None] / 4 * inv).cos(), atol=1e-5)
    nh = R.build_rope_cache_longrope(64, 16, 10000.0, [4.0] * 8, 10)
    assert torch.allclose(nh[:10], c[:10], atol=1e-6) and torch.allclose(nh[10:], pi[10:], atol=1e-6)
    for bad in ([0.5] * 8, [2.0, 1.0] + [2.0] * 6, [1.0] * 7):
        with pytest.raises(ValueError):
            R.build_rope_cache_longrope(8, 16, 10000.0, bad, 0)
    # YaRN: temperature baked into cos and sin, high positions change, low-index dims keep their frequency
    y = R.build_rope_cache(64, 16, 10000.0, scale=4.0, orig_maxpos=16.0)
    m = 0.1 * math.log(4.0) + 1.0
    assert abs(float(y[0, 0]) - m) < 1e-6
    assert not torch.allclose(y[40:] / m, c[40:], atol=1e-3)
    assert torch.allclose(R.build_rope_cache(64, 16, 10000.0, scale=4.0, orig_maxpos=16.0, no_mscale=True)[0, 0], torch.tensor(1.0))


def test_lr_schedules():
    assert lr.cosine_lr(0, 1.0, 0.1, 10, 100) == pytest.approx(0.1)
    assert lr.cosine_lr(9, 1.0, 0.1, 10, 100) == pytest.approx(1.0)
    assert lr.cosine_lr(100, 1.0, 0.1, 10, 100) == pytest.approx(0.1)
    assert lr.cosine_lr(55, 1.0, 0.1, 10, 100) == pytest.approx(0.55)
    base = lr.cosine_lr(60, 0.5, 0.1, 10, 100)
    assert lr.rewarmup_lr(50, 1.0, 0.1, 10, 100, 50, 10, 0.5) == pytest.approx(base / 10)
    assert lr.rewarmup_lr(59, 1.0, 0.1, 10, 100, 50, 10, 0.5) == pytest.approx(base)
    assert lr.rewarmup_lr(70, 1.0, 0.1, 10, 100, 50, 10, 0.5) == pytest.approx(lr.cosine_lr(70, 0.5, 0.1, 10, 100))
    assert lr.rewarmup_lr(70, 1.0, 0.1, 10, 100, -1, 10, 0.5) == lr.cosine_lr(70, 1.0, 0.1, 10, 100)


def test_config_env_surface():
    c = Config.from_env("llama", 4, env={"CP_SIZE": "2", "CP_ATTN_MODE": "ring", "CP_T": "8192", "CP_N_EMBD": "768",
                                         "CP_N_HEAD": "12", "CP_N_KVHEAD": "4", "YARN_SCALE": "4", "CP_ROTATOR": "AllGather",
                                         "CP_RECOMPUTE_K": "1", "CP_CKPT_RESUME": "3"})
    assert (c.cp_size, c.dp_size, c.attn_mode, c.T, c.head_dim, c.ffn_hidden) == (2, 2, "ring", 8192, 64, 2048)
    assert c.yarn.scale == 4.0 and c.rotator == "allgather" and c.recompute_k and c.ckpt_resume == 3 and c.load_balance
    c.validate()
    g = Config.from_env("gpt2", 2, env={"CP_MODEL_44M": "1"})
    assert (g.n_embd, g.n_layer, g.n_head, g.global_batch, g.max_steps, g.warmup_steps) == (384, 3, 6, 65536, 6768, 676)
    assert g.share_fwd_rotator and g.attn_mode == "ring" and g.vocab_padded % 64 == 0
    with pytest.warns(UserWarning):
        Config.from_env("llama", 1, env={"CP_TYPO": "1"})
    with pytest.raises(ValueError):
        Config.from_env("llama", 4, env={"CP_ATTN_MODE": "ulysses", "CP_N_HEAD": "6"}).validate()
    with pytest.raises(ValueError):
        Config.from_env("llama", 4, env={"CP_ATTN_MODE": "hybrid", "CP_ULYSSES_SIZE": "3"}).validate()
    with pytest.raises(ValueError):
        Config.from_env("llama", 2, env={"CP_CREAM_MODE": "cream"}).validate()


def test_mesh_math_native():
    from context_parallelism_b200.parallel import mesh
    assert mesh.mesh_coords((2, 2, 2), 5) == [1, 0, 1]
    assert mesh.mesh_rank((2, 2, 2), [1, 0, 1]) == 5
    assert mesh.mesh_group_ranks((2, 2, 2), 5, 1) == [5, 7]
    assert mesh.mesh_group_ranks((2, 4), 6, 1) == [4, 5, 6, 7]
    assert mesh.mesh_group_ranks((2, 4), 6, 0) == [2, 6]
    m = mesh.DeviceMesh((2, 4), ("dp", "cp"), rank=6, world_size=8, create_groups=False)
    assert (m.coord("dp"), m.coord("cp"), m.ranks("cp")) == (1, 2, [4, 5, 6, 7])
    cfg = Config.from_env("llama", 8, env={"CP_SIZE": "4", "CP_ATTN_MODE": "hybrid", "CP_ULYSSES_SIZE": "2", "CP_RING_OUTER": "1"})
    m = mesh.DeviceMesh.for_config(cfg, 3, 8, create_groups=False)
    assert m.names == ("ring", "dp", "ulysses") and m.shape == (2, 2, 2)


def test_lse_merge_equals_joint_softmax():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 16, 2, 8), torch.randn(1, 32, 2, 8), torch.randn(1, 32, 2, 8)
    o, l = R.attention_dense(q, k, v, 0.3, causal=False)
    o1, l1 = R.attention_dense(q, k[:, :20], v[:, :20], 0.3, causal=False)
    o2, l2 = R.attention_dense(q, k[:, 20:], v[:, 20:], 0.3, causal=False)
    om, lm = R.lse_merge(o1, l1, o2, l2)
    assert torch.allclose(om, o, atol=1e-5) and torch.allclose(lm, l, atol=1e-5)
    ninf = torch.full_like(l2, float("-inf"))
    om, lm = R.lse_merge(o1, l1, torch.zeros_like(o2), ninf)
    assert torch.allclose(om, o1) and torch.allclose(lm, l1)


def test_gamma_grad_accumulation_rule():
    """QK-norm gain gradients: summed locally over ring steps, then AVERAGED over ranks by the parameter
    all-reduce, equal the single-rank gradient when each rank's loss is a mean over its own tokens
    (context_parallel/RopeGammaAccum.h:16-21); a cross-rank SUM would be N times too large."""
    torch.manual_seed(1)
    N, T, D = 2, 8, 4
    x = torch.randn(T, D)
    g = torch.ones(D, requires_grad=True)
    w = torch.randn(T, D)
    (R.rmsnorm(x, g, 1e-6) * w).sum(-1).mean().backward()
    full = g.grad.clone()
    parts = []
    for r in range(N):
        gg = torch.ones(D, requires_grad=True)
        idx = shard.local_positions(T, N, r, True)
        (R.rmsnorm(x[idx], gg, 1e-6) * w[idx]).sum(-1).mean().backward()
        parts.append(gg.grad)
    assert torch.allclose(sum(parts) / N, full, atol=1e-6)
    assert not torch.allclose(sum(parts), full, atol=1e-3)


def test_longrope_factor_file_reference_layout(tmp_path):
    """``n_hat <int>`` / ``s <int>`` / ``S_search <int>`` / ``lambda f0 f1 ...`` tokens in any order, ``#`` comments
    (Scripts/Blutrain/bluscriptCP.cpp:538-572); what the search tool writes is read back unchanged; malformed files
    are refused with the reference's conditions."""
    from context_parallelism_b200.ops import rope as R
    p = tmp_path / "f.txt"
    p.write_text("# GA best\nlambda 1.0 1.25 2.5 4.0   # tail comment\nS_search 32768 n_hat 4\ns 8\n")
    assert R.parse_longrope_factors(str(p), 4) == ([1.0, 1.25, 2.5, 4.0], 4, 8, 32768)
    R.write_longrope_factors(str(p), [1.0, 2.0, 2.0, 3.5], 2, 8, 4096)
    assert p.read_text().split() == ["n_hat", "2", "s", "8", "S_search", "4096", "lambda", "1.000000", "2.000000", "2.000000", "3.500000"]
    assert R.parse_longrope_factors(str(p), 4) == ([1.0, 2.0, 2.0, 3.5], 2, 8, 4096)
    for text in ("lambda 1 2 3 4\n",                      # no n_hat
                 "n_hat 0\nlambda 1 2 3\n",               # too few values
                 "n_hat 0\nlambda 0.5 1 2 3\n",           # below 1
                 "n_hat 0\nlambda 1 3 2 4\n",             # decreasing
                 "n_hat x\nlambda 1 2 3 4\n",             # bad integer
                 "n_hat 0\nfoo 3\nlambda 1 2 3 4\n"):     # unknown token
        p.write_text(text)
        with pytest.raises(ValueError):
            R.parse_longrope_factors(str(p), 4)
    p.write_text("n_hat=1\ns=4\nsearch_len=64\n1.0 2.0 3.0 4.0\n")      # the older key=value form still loads
    assert R.parse_longrope_factors(str(p), 4) == ([1.0, 2.0, 3.0, 4.0], 1, 4, 64)


# ----------------------------------------------------------------------------- sharded optimiser plan
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_shard_plan_partitions_every_bucket(world):
    """Every flat index has exactly one owner, owner boundaries are multiples of 8 elements, the shard buffers of one rank
    are the concatenation of its padded runs, and the device kernels' ownership rule (element offset inside the bucket divided
    by ``per``: csrc/kernels/comm.cu, reduce_scatter_f32_kernel / allgather_pull_kernel) names the same owner."""
    from context_parallelism_b200.ops.optim import ShardPlan, plan_buckets
    sizes = [64 * 3, 64 * 10, 64, 64 * 7, 64 * 2, 64 * 33]
    entries, off = [], 0
    for i, n in enumerate(sizes):
        entries.append((f"p{i}", None, off, n))
        off += n
    buckets = plan_buckets(entries, off, bucket_elems=64 * 9)
    assert buckets[0][0] == 0 and buckets[-1][1] == off
    assert all(a[1] == b[0] for a, b in zip(buckets, buckets[1:]))             # contiguous, cut at parameter boundaries
    owner = [-1] * off
    for r in range(world):
        plan = ShardPlan(buckets, world, r)
        runs = plan.owned()
        assert runs == sorted(runs)
        for a, c, sb in runs:
            assert a % 8 == 0 and sb % 8 == 0 and 0 <= sb and sb + (c - a) <= plan.shard_total
            for e in range(a, c):
                assert owner[e] == -1
                owner[e] = r
        for (s, n, per, shard_off), (a, c, sb) in zip([b for b in plan.buckets if b[0] + r * b[2] < b[0] + b[1]], runs):
            assert per % 8 == 0 and per * world >= n and sb == shard_off and a == s + r * per
    assert all(o >= 0 for o in owner)
    plan = ShardPlan(buckets, world, 0)
    for s, n, per, _ in plan.buckets:
        for e in range(s, s + n, 5):
            assert owner[e] == (e - s) // per


@pytest.mark.parametrize("N", [1, 2, 4, 8])
@pytest.mark.parametrize("lb", [True, False])
def test_ring_chunk_tables_are_inverse(N, lb):
    """``ring_rank_chunks`` and ``ring_chunk_owner`` describe the same assignment of the 2N position-ordered chunks
    (head-tail balanced: rank r holds chunks r and 2N-1-r, context_parallel/HeadTailLoadBalancer.h:46-64; contiguous: 2r, 2r+1)."""
    from context_parallelism_b200.parallel.fused import ring_chunk_owner, ring_rank_chunks
    seen = set()
    for r in range(N):
        chunks = ring_rank_chunks(r, N, lb)
        assert len(chunks) == 2
        for half, c in enumerate(chunks):
            assert ring_chunk_owner(c, N, lb) == (r, half)
            seen.add(c)
    assert seen == set(range(2 * N))
    if lb:
        # causal work per rank is equal: chunk c attends to c + 1 chunks (itself included)
        work = [sum(c + 1 for c in ring_rank_chunks(r, N, True)) for r in range(N)]
        assert len(set(work)) == 1


@pytest.mark.parametrize("m_tiles,n_blocks,band", [(1, 1, 8), (11, 32, 8), (64, 8, 8), (5, 3, 1), (9, 7, 4), (32, 32, 8)])
def test_pair_gemm_band_order_visits_every_tile_once(m_tiles, n_blocks, band):
    """The tile order of the CTA-pair GEMM (csrc/kernels/gemm2.cu, pair_tile_coords): bands of ``band`` pair-rows swept along
    N with rows fastest, the last band possibly shorter.  Restated here; the device code is checked against cuBLAS-free fp32
    matmul on a ragged shape in tests/test_gpu_kernels.py::test_gemm_pair_banded_order."""
    def coords(tile):
        per_band = band * n_blocks
        b, idx = divmod(tile, per_band)
        rows = min(band, m_tiles - b * band)
        nb, r = divmod(idx, rows)
        return b * band + r, nb
    got = [coords(t) for t in range(m_tiles * n_blocks)]
    assert sorted(got) == [(m, n) for m in range(m_tiles) for n in range(n_blocks)]
    # consecutive tiles of a full band share a column of B (rows fastest)
    if m_tiles >= band > 1:
        assert [c[1] for c in got[:band]] == [0] * band and [c[0] for c in got[:band]] == list(range(band))
