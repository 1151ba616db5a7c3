"""Numerics of each sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

from util import assert_close

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda", 0)


def check_status():
    from context_parallelism_b200 import _native as nv
    torch.cuda.synchronize()
    nv.status_for(dev()).check()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1000, 384, 520), (4096, 2048, 2048), (72, 128, 64)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_majors(M, N, K, a_mn, b_mn):
    from context_parallelism_b200.ops.gemm import gemm
    torch.manual_seed(0)
    A = torch.randn(M, K, device=dev()).bfloat16()
    B = torch.randn(N, K, device=dev()).bfloat16()
    want = A.float() @ B.float().t()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    got = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    check_status()
    assert_close(got.float(), want, cos=0.9999, rel=2e-2, name=f"gemm {M}x{N}x{K} a_mn={a_mn} b_mn={b_mn}")


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_pair_banded_order(a_mn, b_mn):
    """A B operand above 64 MB switches the CTA-pair kernel to its banded tile order (8 pair-rows per band, a ragged last
    band here: 11 pair-rows); every output tile must still be produced exactly once."""
    from context_parallelism_b200.ops.gemm import gemm
    torch.manual_seed(3)
    M, N, K = 2816 - 8, 8192, 4160
    A = torch.randn(M, K, device=dev()).bfloat16()
    B = (torch.randn(N, K, device=dev()) * 0.1).bfloat16()
    want = A.float() @ B.float().t()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    got = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    check_status()
    assert_close(got.float(), want, cos=0.9999, rel=2e-2, name=f"banded gemm a_mn={a_mn} b_mn={b_mn}")


def test_gemm_epilogues():
    from context_parallelism_b200.ops import gemm as G
    torch.manual_seed(1)
    M, N, K = 512, 768, 384
    A = torch.randn(M, K, device=dev()).bfloat16()
    B = (torch.randn(N, K, device=dev()) * 0.05).bfloat16()
    bias = torch.randn(N, device=dev())
    ref = A.float() @ B.float().t()
    got = G.gemm(A, B, out_dtype=torch.float32, bias=bias)
    assert_close(got, ref + bias, cos=0.99999, rel=1e-3, name="f32+bias")
    acc = torch.ones(M, N, device=dev())
    G.gemm(A, B, out=acc, accumulate=True)
    assert_close(acc, ref + 1, cos=0.99999, rel=1e-3, name="f32 accumulate")
    pre = torch.empty(M, N, device=dev(), dtype=torch.bfloat16)
    act = G.gemm(A, B, bias=bias, epi=G.EPI_BF16_GELU, aux=pre)
    assert_close(pre.float(), ref + bias, cos=0.9999, rel=2e-2, name="gelu pre")
    assert_close(act.float(), torch.nn.functional.gelu(ref + bias, approximate="tanh"), cos=0.9999, rel=2e-2, name="gelu")
    Fh = N // 2
    gu = torch.empty(M, N, device=dev(), dtype=torch.bfloat16)
    sw = G.gemm(A, B, epi=G.EPI_BF16_SWIGLU, aux=gu)
    assert sw.shape == (M, Fh)
    assert_close(gu.float(), ref, cos=0.9999, rel=2e-2, name="swiglu pre")
    assert_close(sw.float(), torch.nn.functional.silu(ref[:, :Fh]) * ref[:, Fh:], cos=0.9999, rel=3e-2, name="swiglu")
    check_status()


def test_linear_autograd():
    from context_parallelism_b200.ops.gemm import linear, linear_swiglu, linear_gelu
    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device=dev()).bfloat16().requires_grad_()
    w = (torch.randn(512, 256, device=dev()) * 0.05).bfloat16().requires_grad_()
    b = torch.randn(512, device=dev(), requires_grad=True)
    for fn, rf in ((lambda: linear(x, w, b), lambda X, W, Bb: torch.nn.functional.linear(X, W, Bb)),
                   (lambda: linear_gelu(x, w, b), lambda X, W, Bb: torch.nn.functional.gelu(torch.nn.functional.linear(X, W, Bb), approximate="tanh")),
                   (lambda: linear_swiglu(x, w), lambda X, W, Bb: torch.nn.functional.silu(torch.nn.functional.linear(X, W)[..., :256]) * torch.nn.functional.linear(X, W)[..., 256:])):
        x.grad = w.grad = b.grad = None
        y = fn()
        dy = torch.randn_like(y)
        y.backward(dy)
        X, W, Bb = x.detach().float().requires_grad_(), w.detach().float().requires_grad_(), b.detach().clone().requires_grad_()
        Y = rf(X, W, Bb)
        Y.backward(dy.float())
        assert_close(y.float(), Y, cos=0.9999, name="fwd")
        assert_close(x.grad.float(), X.grad, cos=0.999, name="dx")
        assert_close(w.grad.float(), W.grad, cos=0.999, name="dw")
        if Bb.grad is not None and b.grad is not None:
            assert_close(b.grad.float(), Bb.grad, cos=0.999, name="db")
    check_status()


@pytest.mark.parametrize("layer", [0, 1])
@pytest.mark.parametrize("d", [384, 768, 2048, 4096])
@pytest.mark.parametrize("with_res", [False, True])
def test_norm(layer, d, with_res):
    from context_parallelism_b200.ops import elementwise as E
    torch.manual_seed(3)
    rows = 300
    x = torch.randn(rows, d, device=dev()).bfloat16().requires_grad_()
    r = torch.randn(rows, d, device=dev()).bfloat16().requires_grad_() if with_res else None
    w = (1 + 0.1 * torch.randn(d, device=dev())).requires_grad_()
    b = (0.1 * torch.randn(d, device=dev())).requires_grad_() if layer else None
    y, xn = (E.layernorm(x, w, b, 1e-5, r) if layer else E.rmsnorm(x, w, 1e-5, r))
    dy, dxn = torch.randn_like(y), torch.randn_like(y)
    (y.float() * dy.float()).sum().backward() if False else torch.autograd.backward([y, xn], [dy, dxn])
    X = x.detach().float().requires_grad_()
    R = r.detach().float().requires_grad_() if with_res else None
    W = w.detach().clone().requires_grad_()
    Bb = b.detach().clone().requires_grad_() if layer else None
    XN = (X + R).bfloat16().float() if with_res else X
    if with_res:
        XN = X + R
    if layer:
        Y = torch.nn.functional.layer_norm(XN, (d,), W, Bb, 1e-5)
    else:
        Y = XN * torch.rsqrt(XN.pow(2).mean(-1, keepdim=True) + 1e-5) * W
    torch.autograd.backward([Y, XN], [dy.float(), dxn.float()])
    assert_close(y.float(), Y, cos=0.9999, rel=3e-2, name="y")
    assert_close(x.grad.float(), X.grad, cos=0.999, name="dx")
    if with_res:
        assert_close(r.grad.float(), R.grad, cos=0.999, name="dres")
    assert_close(w.grad, W.grad, cos=0.999, name="dw")
    if layer:
        assert_close(b.grad, Bb.grad, cos=0.999, name="db")


@pytest.mark.parametrize("D", [64, 128])
def test_qk_norm_rope(D):
    from context_parallelism_b200.ops import elementwise as E, reference as R
    torch.manual_seed(4)
    B, T, Hq, Hkv = 2, 96, 4, 2
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, device=dev()).bfloat16().requires_grad_()
    gq = (1 + 0.1 * torch.randn(D, device=dev())).requires_grad_()
    gk = (1 + 0.1 * torch.randn(D, device=dev())).requires_grad_()
    cache = R.build_rope_cache(512, D, 10000.0).to(dev())
    pos = torch.randint(0, 512, (T,), device=dev())
    out = E.qk_norm_rope(qkv, gq, gk, cache, pos, Hq, Hkv, D, 1e-6)
    dout = torch.randn_like(out)
    out.backward(dout)
    X = qkv.detach().float().cpu().requires_grad_()
    GQ, GK = gq.detach().cpu().requires_grad_(), gk.detach().cpu().requires_grad_()
    want = E.qk_norm_rope(X, GQ, GK, cache.cpu(), pos.cpu(), Hq, Hkv, D, 1e-6)
    want.backward(dout.float().cpu())
    assert_close(out.float().cpu(), want, cos=0.9999, rel=3e-2, name="fwd")
    assert_close(qkv.grad.float().cpu(), X.grad, cos=0.999, name="dqkv")
    assert_close(gq.grad.cpu(), GQ.grad, cos=0.999, name="dgq")
    assert_close(gk.grad.cpu(), GK.grad, cos=0.999, name="dgk")
    check_status()


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("B,Tq,Tk,Hq,Hkv,causal", [
    (1, 128, 128, 1, 1, False), (1, 128, 128, 1, 1, True), (2, 384, 384, 4, 2, True),
    (1, 200, 328, 2, 1, False), (1, 1024, 1024, 2, 2, True)])
def test_flash_fwd(D, B, Tq, Tk, Hq, Hkv, causal):
    from context_parallelism_b200.ops import attention as A, reference as R
    torch.manual_seed(5)
    q = torch.randn(B, Tq, Hq, D, device=dev()).bfloat16()
    k = torch.randn(B, Tk, Hkv, D, device=dev()).bfloat16()
    v = torch.randn(B, Tk, Hkv, D, device=dev()).bfloat16()
    scale = 1 / math.sqrt(D)
    out, lse = A.flash_fwd(q, k, v, scale, causal)
    check_status()
    want, wlse = R.attention_dense(q.float(), k.float(), v.float(), scale, causal=causal)
    assert_close(out.float(), want, cos=0.9995, rel=3e-2, name="out")
    assert_close(lse, wlse, cos=0.99999, rel=1e-3, name="lse")


def test_flash_fwd_positions_packed():
    """Global-position masking with a HeadTail query shard against a position-ordered K/V, consumed as
    strided views of a packed QKV buffer."""
    from context_parallelism_b200.ops import attention as A, reference as R
    from context_parallelism_b200.parallel.shard import local_positions
    torch.manual_seed(6)
    B, T, Hq, Hkv, D, N, r = 1, 1024, 4, 2, 64, 4, 1
    qkv = torch.randn(B, T, (Hq + 2 * Hkv), D, device=dev()).bfloat16()
    qfull, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    pos = local_positions(T, N, r, True).to(dev())
    q = qfull[:, pos].contiguous()
    out, lse = A.flash_fwd(q, k, v, 0.125, True, q_pos=pos.int())
    check_status()
    want, wlse = R.attention_dense(q.float(), k.float(), v.float(), 0.125, q_pos=pos, causal=True)
    assert_close(out.float(), want, cos=0.9995, rel=3e-2, name="out")
    assert_close(lse, wlse, cos=0.99999, rel=1e-3, name="lse")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("B,Tq,Tk,Hq,Hkv,causal", [
    (1, 128, 128, 1, 1, False), (1, 128, 128, 1, 1, True), (2, 384, 384, 4, 2, True),
    (1, 200, 328, 2, 1, False), (1, 1024, 1024, 4, 1, True)])
def test_flash_bwd(D, B, Tq, Tk, Hq, Hkv, causal):
    from context_parallelism_b200.ops import attention as A, reference as R
    torch.manual_seed(7)
    q = torch.randn(B, Tq, Hq, D, device=dev()).bfloat16()
    k = torch.randn(B, Tk, Hkv, D, device=dev()).bfloat16()
    v = torch.randn(B, Tk, Hkv, D, device=dev()).bfloat16()
    do = torch.randn(B, Tq, Hq, D, device=dev()).bfloat16()
    scale = 1 / math.sqrt(D)
    out, lse = A.flash_fwd(q, k, v, scale, causal)
    dq, dk, dv = A.flash_bwd(q, k, v, out, lse, do, scale, causal)
    check_status()
    want, wlse = R.attention_dense(q.float(), k.float(), v.float(), scale, causal=causal)
    wdq, wdk, wdv = R.attention_dense_bwd(q.float(), k.float(), v.float(), want, wlse, do.float(), scale, causal=causal)
    assert_close(dv.float(), wdv, cos=0.998, rel=5e-2, name="dv")
    assert_close(dk.float(), wdk, cos=0.998, rel=5e-2, name="dk")
    assert_close(dq.float(), wdq, cos=0.998, rel=5e-2, name="dq")


@pytest.mark.parametrize("B,Tq,Tk,Hq,Hkv,causal", [(1, 512, 512, 4, 1, True), (2, 300, 712, 2, 2, False), (1, 2048, 2048, 8, 2, True)])
def test_flash_bwd_d64_kernels_agree(B, Tq, Tk, Hq, Hkv, causal, monkeypatch):
    """The head_dim-64 kernel (transposed, vectors folded into the MMAs) against the general kernel on the same inputs,
    including the fp32-accumulating dK/dV mode; query positions of a zig-zag shard when causal."""
    from context_parallelism_b200.ops import attention as A, attention_bwd as AB
    from context_parallelism_b200.parallel.shard import local_positions
    torch.manual_seed(11)
    D = 64
    q = torch.randn(B, Tq, Hq, D, device=dev()).bfloat16()
    k = torch.randn(B, Tk, Hkv, D, device=dev()).bfloat16()
    v = torch.randn(B, Tk, Hkv, D, device=dev()).bfloat16()
    do = torch.randn(B, Tq, Hq, D, device=dev()).bfloat16()
    scale = 1 / math.sqrt(D)
    q_pos = None
    if causal and Tq == 512:
        q_pos = local_positions(4 * Tq, 4, 1, True).to(dev()).int()       # rank 1 of 4: chunks 1 and 6
        k = torch.randn(B, 4 * Tq, Hkv, D, device=dev()).bfloat16()
        v = torch.randn_like(k)
    out, lse = A.flash_fwd(q, k, v, scale, causal, q_pos=q_pos)
    got = {}
    for general in (True, False):
        monkeypatch.setattr(AB, "_USE_GENERAL_D64", general)
        got[general] = A.flash_bwd(q, k, v, out, lse, do, scale, causal, q_pos=q_pos)
        check_status()
    for a, b_, n in zip(got[True], got[False], ("dq", "dk", "dv")):
        assert torch.isfinite(b_.float()).all()
        assert_close(b_.float(), a.float(), cos=0.9995, rel=3e-2, name=n)


def test_flash_autograd_positions():
    from context_parallelism_b200.ops import attention as A
    from context_parallelism_b200.parallel.shard import local_positions
    torch.manual_seed(8)
    B, T, Hq, Hkv, D, N, r = 1, 1024, 4, 2, 64, 4, 2
    pos = local_positions(T, N, r, True).to(dev())
    q = torch.randn(B, T // N, Hq, D, device=dev()).bfloat16().requires_grad_()
    k = torch.randn(B, T, Hkv, D, device=dev()).bfloat16().requires_grad_()
    v = torch.randn(B, T, Hkv, D, device=dev()).bfloat16().requires_grad_()
    out, _ = A.flash_attention(q, k, v, None, True, pos.int())
    do = torch.randn_like(out)
    out.backward(do)
    check_status()
    Q, K, V = (t.detach().float().cpu().requires_grad_() for t in (q, k, v))
    want, _ = A.flash_attention(Q, K, V, None, True, pos.cpu())
    want.backward(do.float().cpu())
    assert_close(out.float().cpu(), want, cos=0.9995, name="out")
    for a, b_, n in ((q, Q, "dq"), (k, K, "dk"), (v, V, "dv")):
        assert_close(a.grad.float().cpu(), b_.grad, cos=0.998, name=n)


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 4, 2), (128, 2, 1), (32, 4, 4)])
def test_attention_fp32_accurate_variant(D, Hq, Hkv):
    """ATTN_FP32 kernels: fp32 arithmetic on bf16 inputs reproduces the dense oracle far more tightly than the tensor-core
    path (forward cos > 0.99999 and 1e-3 relative, gradients cos > 0.9999: the reference's fp32 bars)."""
    from context_parallelism_b200.ops import attention as A
    from context_parallelism_b200.ops import reference as ref
    torch.manual_seed(3)
    B, T = 2, 200
    q, k, v, do = (torch.randn(B, T, h, D, device=dev()).bfloat16() for h in (Hq, Hkv, Hkv, Hq))
    scale = D ** -0.5
    qpos = torch.arange(T, device=dev()) + 7
    A.FP32_ACCURATE = True
    try:
        qi, ki, vi = (t.clone().requires_grad_() for t in (q, k, v))
        o, lse = A.flash_attention(qi, ki, vi, scale, True, qpos, 5)
        o.backward(do)
    finally:
        A.FP32_ACCURATE = False
    kp = torch.arange(5, 5 + T, device=dev())
    o_ref, lse_ref = ref.attention_dense(q.float(), k.float(), v.float(), scale, qpos, kp, True)
    g_ref = ref.attention_dense_bwd(q.float(), k.float(), v.float(), o_ref, lse_ref, do.float(), scale, qpos, kp, True)
    check_status()
    assert_close(o.float(), o_ref, cos=0.99999, rel=1e-2, name="fp32 attn out")       # the bf16 rounding of the output remains
    assert_close(lse, lse_ref, cos=0.999999, rel=1e-4, name="fp32 attn lse")
    for got, want, nm in zip((qi.grad, ki.grad, vi.grad), g_ref, ("dq", "dk", "dv")):
        assert_close(got.float(), want, cos=0.9999, rel=2e-2, name="fp32 attn " + nm)
