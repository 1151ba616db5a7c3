"""Stand-alone timing of the sm_100a kernels with CUDA events: attention forward / backward (TFLOP/s), the GEMM in
its three layouts against ``torch.matmul`` (cuBLAS) in the same process, and the memory-bound kernels as algorithmic
bytes over time against the measured copy bandwidth.

Hygiene: 3 warm-up launches, every timed launch preceded by a write of a 256 MB buffer (larger than the 126 MB L2) on
the same stream *outside* the event pair, events on the launching stream, one synchronisation per measurement.  The
row-wise memory-bound kernels are reached through autograd functions whose host path is comparable to their run time, so
their event pair sits directly around the kernel launch (``Timer.kernel_ms``).  The
denominators come from ``MEASURED_PEAKS.json`` at the repository root when present (``--peaks`` overrides), else the
fallback 6650 GB/s and 1590 TFLOP/s.

    python -m context_parallelism_b200.experiments.kernel_bench --what attn gemm membound
"""
from __future__ import annotations

import argparse
import json
import math
import os
from pathlib import Path

import torch


def _peaks(path):
    for p in ([path] if path else []) + [str(Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json")]:
        if p and os.path.exists(p):
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self, dev, flush_mb=256):
        self.dev = dev
        self.flush = torch.empty(flush_mb << 20, dtype=torch.uint8, device=dev)

    def ms(self, fn, iters=5, warm=3, flush=True):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        pairs = []
        for _ in range(iters):
            if flush:
                self.flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            pairs.append((e0, e1))
        torch.cuda.synchronize()
        t = sorted(a.elapsed_time(b) for a, b in pairs)
        return t[len(t) // 2]

    def kernel_ms(self, fn, name, iters=5, warm=3):
        """Device time of the launches of kernel ``name`` inside one call of ``fn`` (an event pair around each launch on
        its own stream, see ``_native.profile_start``): what ``ms`` would show if the host could launch instantly.  For
        calls that go through autograd the host path is a sizeable part of ``ms``."""
        from context_parallelism_b200 import _native as nv
        for _ in range(warm):
            fn()
        t = []
        for _ in range(iters):
            self.flush.fill_(1)
            nv.profile_start()
            fn()
            t.append(nv.profile_stop()[name][1])
        t.sort()
        return t[len(t) // 2]


def bench_attention(tm, out, shapes, tflops_peak, which="both"):
    from context_parallelism_b200.ops import attention as A
    for D, Hq, Hkv, T in shapes:
        dev = tm.dev
        q = torch.randn(1, T, Hq, D, device=dev).bfloat16()
        k = torch.randn(1, T, Hkv, D, device=dev).bfloat16()
        v = torch.randn_like(k)
        sc = 1 / math.sqrt(D)
        if which in ("both", "fwd"):
            ms = tm.ms(lambda: A.flash_fwd(q, k, v, sc, True))
            fl = 4 * T * T * Hq * D / 2
            out.append({"kernel": "flash_fwd", "head_dim": D, "heads": f"{Hq}/{Hkv}", "T": T, "ms": ms, "tflops": fl / ms / 1e9,
                        "frac_of_peak": fl / ms / 1e9 / tflops_peak})
        if which == "fwd":
            continue
        o, lse = A.flash_fwd(q, k, v, sc, True)
        do = torch.randn_like(o)
        ms = tm.ms(lambda: A.flash_bwd(q, k, v, o, lse, do, sc, True))
        fl = 10 * T * T * Hq * D / 2
        out.append({"kernel": "flash_bwd (prep + core + dq cast)", "head_dim": D, "heads": f"{Hq}/{Hkv}", "T": T, "ms": ms,
                    "tflops": fl / ms / 1e9, "frac_of_peak": fl / ms / 1e9 / tflops_peak})


def bench_gemm(tm, out, shapes, tflops_peak):
    from context_parallelism_b200.ops import gemm as G
    dev = tm.dev
    for M, N, K in shapes:
        a = torch.randn(M, K, device=dev).bfloat16()
        b = torch.randn(N, K, device=dev).bfloat16()
        at, bt = a.t().contiguous(), b.t().contiguous()
        fl = 2.0 * M * N * K
        lib = tm.ms(lambda: torch.matmul(a, b.t()))
        for name, fn in (("NT (forward)", lambda: G.gemm(a, b)), ("NN (data gradient)", lambda: G.gemm(a, bt, b_mn=True)),
                         ("TN (weight gradient)", lambda: G.gemm(at, bt, a_mn=True, b_mn=True))):
            ms = tm.ms(fn)
            out.append({"kernel": "gemm_bf16 " + name, "M": M, "N": N, "K": K, "ms": ms, "tflops": fl / ms / 1e9,
                        "frac_of_peak": fl / ms / 1e9 / tflops_peak, "vs_cublas": lib / ms, "cublas_tflops": fl / lib / 1e9})


def bench_membound(tm, out, rows, d, hbm_gbs):
    """Algorithmic bytes (every input read once, every output written once) over CUDA-event time."""
    from context_parallelism_b200 import _native as nv
    from context_parallelism_b200.ops import elementwise as E
    from context_parallelism_b200.ops import xent as X
    dev = tm.dev
    x = torch.randn(rows, d, device=dev).bfloat16()
    res = torch.randn_like(x)
    w = torch.ones(d, device=dev)

    def rec(name, ms, nbytes, **kw):
        out.append(dict({"kernel": name, "rows": rows, "d": d, "ms": ms, "algorithmic_MB": nbytes / 1e6,
                         "GBps": nbytes / ms / 1e6, "frac_of_copy_bw": nbytes / ms / 1e6 / hbm_gbs}, **kw))
    with torch.no_grad():
        ms = tm.kernel_ms(lambda: E.rmsnorm(x, w, 1e-5, res), "norm_fwd")
        rec("norm_fwd (rmsnorm + residual)", ms, rows * d * 2 * 4 + rows * 8)          # x, res in; x_new, y out; stats
    xr = x.clone().requires_grad_()
    y, xn = E.rmsnorm(xr, w, 1e-5, res)
    dy = torch.randn_like(y)
    w.main_grad = torch.zeros(d, device=dev)

    def nb():
        torch.autograd.grad([y, xn], [xr], [dy, dy], retain_graph=True)
    ms = tm.kernel_ms(nb, "norm_bwd")
    rec("norm_bwd (rmsnorm, two upstream gradients)", ms, rows * d * 2 * 4 + rows * 8)  # x_new, dy, dres in; dx out
    # QK-norm + RoPE over a packed QKV row of the 1B shape (32 + 2*8 heads of 64)
    Hq, Hkv, D = 32, 8, 64
    T = rows
    qkv = torch.randn(1, T, (Hq + 2 * Hkv) * D, device=dev).bfloat16()
    from context_parallelism_b200.ops import rope as R
    cache = R.build_rope_cache(T, D, 5e5, dev, None)
    pos = torch.arange(T, device=dev)
    g = torch.ones(D, device=dev)
    with torch.no_grad():
        ms = tm.kernel_ms(lambda: E.qk_norm_rope(qkv, g, g, cache, pos, Hq, Hkv, D, 1e-6), "qk_norm_rope_fwd")
    rec("qk_norm_rope_fwd", ms, T * (Hq + 2 * Hkv) * D * 2 * 2 + T * D * 4)
    # SwiGLU backward: pre-activation [rows, 2F] and dact [rows, F] in, d(pre) [rows, 2F] out
    F_ = 4 * d
    gu = torch.randn(rows, 2 * F_, device=dev).bfloat16()
    dact = torch.randn(rows, F_, device=dev).bfloat16()
    ms = tm.ms(lambda: E.swiglu_bwd(gu, dact))
    rec("swiglu_bwd", ms, rows * F_ * 2 * 5)
    # cross entropy over one fp32 logit chunk: logits in, bf16 dlogits out
    V = 128256
    cr = min(rows, 4096)
    logits = torch.randn(cr, V, device=dev)
    tg = torch.randint(0, V, (cr,), device=dev)
    ls = torch.zeros(1, device=dev)
    ms = tm.kernel_ms(lambda: X.xent_chunk(logits, tg, ls, 1.0, True, None, V), "xent")
    rec("xent (loss + bf16 dlogits)", ms, cr * V * (4 + 2), rows=cr, d=V)
    # AdamW: p, g, m, v read; p, m, v, bf16 copy written
    n = 256 << 20
    p, gr, m, v = (torch.randn(n, device=dev) * 0.01 for _ in range(4))
    v.abs_()
    p16 = torch.empty(n, dtype=torch.bfloat16, device=dev)
    ssq = torch.ones(1, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    ms = tm.ms(lambda: nv.call("adamw", nv.ptr(p), nv.ptr(gr), nv.ptr(m), nv.ptr(v), nv.ptr(p16), nv.l(n), nv.f(1e-3), nv.f(0.9),
                               nv.f(0.95), nv.f(1e-8), nv.f(0.1), nv.i(3), nv.f(1.0), nv.f(1.0), nv.ptr(ssq), nv.ptr(flag),
                               nv.stream_ptr(dev)))
    rec("adamw (clip + decay + bf16 copy)", ms, n * (16 + 12 + 2), rows=n, d=1)
    scratch = torch.zeros(1032, device=dev)
    ticket = torch.zeros(1, dtype=torch.int32, device=dev)
    ms = tm.ms(lambda: nv.call("sumsq", nv.ptr(gr), nv.l(n), nv.ptr(scratch), nv.ptr(ticket), nv.ptr(ssq), nv.stream_ptr(dev)))
    rec("sumsq (gradient norm)", ms, n * 4, rows=n, d=1)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", nargs="+", default=["attn", "gemm", "membound"], choices=["attn", "gemm", "membound"])
    ap.add_argument("--T", type=int, nargs="+", default=[16384])
    ap.add_argument("--head-dims", type=int, nargs="+", default=[64, 128])
    ap.add_argument("--attn-pass", default="both", choices=["both", "fwd", "bwd"])
    ap.add_argument("--gemm-shape", type=int, nargs=3, default=None, metavar=("M", "N", "K"), help="time this one GEMM shape only")
    ap.add_argument("--rows", type=int, default=131072, help="token rows of the memory-bound kernels (large enough that a launch "
                                                              "lasts several times the host's launch path)")
    ap.add_argument("--peaks", default="")
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm, tfl, src = _peaks(a.peaks)
    tm = Timer(dev)
    rows = []
    if "attn" in a.what:
        bench_attention(tm, rows, [(D, Hq, Hkv, T) for T in a.T for D, Hq, Hkv in ((64, 32, 8), (128, 16, 4)) if D in a.head_dims], tfl,
                        a.attn_pass)
    if "gemm" in a.what:
        # 8192^3 and the Llama-1B layer shapes at 16384 local tokens: QKV / O projection, gate_up, down
        shapes = [tuple(a.gemm_shape)] if a.gemm_shape else [(8192, 8192, 8192), (16384, 3072, 2048), (16384, 2048, 2048),
                                                              (16384, 16384, 2048), (16384, 2048, 8192)]
        bench_gemm(tm, rows, shapes, tfl)
    if "membound" in a.what:
        bench_membound(tm, rows, a.rows, 2048, hbm)
    from context_parallelism_b200 import _native as nv
    nv.status_for(dev).check("kernel_bench")
    hdr = {"peaks": src, "hbm_gbs": hbm, "bf16_tflops": tfl}
    print(json.dumps(hdr))
    for r in rows:
        print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in r.items()}))
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"header": hdr, "rows": rows}, f, indent=1)


if __name__ == "__main__":
    main()
