"""Kernel micro-benchmarks: ``python -m ferrotorch_b200.utils.kbench [gemm|attn|elementwise|all] [--json out.json]``.

Each case is timed with CUDA events on the launching stream after warm-up, with a buffer larger than L2
written between timed iterations, and reported against the measured peaks of the machine
(``MEASURED_PEAKS.json`` at the repository root when present, else 6.65 TB/s and 1.59 PFLOP/s).
The library number printed beside each case (torch.matmul = cuBLAS, SDPA) is the baseline to beat.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "src": "fallback"}


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    _flush.zero_()


def time_fn(fn, iters=10, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def bench_gemm(results):
    from ferrotorch_b200 import ops
    pk = peaks()
    shapes = [  # (M, N, K, a_mn, b_mn, label)
        (8192, 8192, 8192, False, False, "8192^3 NT"),
        (4096, 6144, 4096, False, False, "llama qkv fwd"),
        (4096, 4096, 4096, False, False, "llama o fwd"),
        (4096, 28672, 4096, False, False, "llama gate_up fwd"),
        (4096, 4096, 14336, False, False, "llama down fwd"),
        (4096, 14336 * 2, 4096, False, True, "dgrad-shaped (b_mn)"),
        (28672, 4096, 4096, True, True, "llama gate_up wgrad"),
        (4096, 128256, 4096, False, False, "lm_head fwd"),
    ]
    for M, N, K, a_mn, b_mn, label in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        from ferrotorch_b200 import _lib
        tail = os.environ.get("FT_GEMM_TAIL") == "1"     # opt-in: the same launch with the last round of tiles cut into K slices
        if tail:
            _lib.call("ft_gemm_set_tail", 0)             # the variable switches the slices on from the first launch: time the plain schedule first
        med, best = time_fn(lambda: ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out))
        nmed = None
        if tail:
            nmed = med
            _lib.call("ft_gemm_set_tail", 1)
            med, best = time_fn(lambda: ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out))
        A = a.t() if a_mn else a
        Bm = b if b_mn else b.t()
        lmed, lbest = time_fn(lambda: torch.matmul(A, Bm, out=out))
        fl = 2.0 * M * N * K
        r = {"case": f"gemm {label} M{M} N{N} K{K}", "ms_median": med, "ms_best": best, "tflops": fl / med / 1e9,
             "tflops_best": fl / best / 1e9, "frac_of_peak": fl / best / 1e9 / pk["bf16_tflops"], "peak_src": pk["src"],
             "ms_median_without_tail_slices": nmed, "cublas_ms_median": lmed, "cublas_tflops": fl / lmed / 1e9, "speedup_vs_cublas": lmed / med}
        results.append(r)
        print(json.dumps(r), flush=True)
        del a, b, out


def bench_attn(results):
    from ferrotorch_b200 import ops
    import math
    pk = peaks()
    for B, S, Hq, Hkv, D in [(1, 4096, 32, 8, 128), (2, 8192, 32, 8, 128), (8, 2048, 8, 1, 128)]:
        qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
        fl = 4.0 * B * Hq * S * S * D / 2
        be = ops.attention.backend()
        med, best = time_fn(lambda: ops.flash_fwd(qkv, B, S, Hq, Hkv, D, True))
        out, lse = ops.flash_fwd(qkv, B, S, Hq, Hkv, D, True)
        do = torch.randn_like(out)
        bmed, bbest = time_fn(lambda: ops.flash_bwd(qkv, out, lse, do, B, S, Hq, Hkv, D, True))
        q = qkv[:, : Hq * D].reshape(B, S, Hq, D).transpose(1, 2)
        k = qkv[:, Hq * D: (Hq + Hkv) * D].reshape(B, S, Hkv, D).transpose(1, 2)
        v = qkv[:, (Hq + Hkv) * D:].reshape(B, S, Hkv, D).transpose(1, 2)
        lmed, _ = time_fn(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True))
        r = {"case": f"attn causal B{B} S{S} Hq{Hq} Hkv{Hkv} D{D}", "backend": be, "fwd_ms": med, "fwd_tflops": fl / med / 1e9,
             "bwd_ms": bmed, "bwd_tflops": 2.5 * fl / bmed / 1e9, "sdpa_fwd_ms": lmed, "frac_of_peak_fwd": fl / best / 1e9 / pk["bf16_tflops"]}
        results.append(r)
        print(json.dumps(r), flush=True)


def bench_elementwise(results):
    from ferrotorch_b200 import ops
    pk = peaks()
    T, d, F, V = 4096, 4096, 14336, 128256
    x = torch.randn(T, d, device="cuda").to(torch.bfloat16)
    w = torch.ones(d, device="cuda", dtype=torch.bfloat16)
    cases = []
    cases.append(("rmsnorm_fwd 4096x4096", lambda: ops.rmsnorm_fwd(x, w, 1e-5), 2 * T * d * 2))
    y, rstd, _ = ops.rmsnorm_fwd(x, w, 1e-5)
    cases.append(("rmsnorm_bwd 4096x4096", lambda: ops.rmsnorm_bwd(x, w, y, rstd), 3 * T * d * 2))
    gu = torch.randn(T, 2 * F, device="cuda").to(torch.bfloat16)
    cases.append(("swiglu_fwd 4096x14336", lambda: ops.swiglu_fwd(gu), 3 * T * F * 2))
    da = torch.randn(T, F, device="cuda").to(torch.bfloat16)
    cases.append(("swiglu_bwd 4096x14336", lambda: ops.swiglu_bwd(gu, da), 5 * T * F * 2))
    logits = torch.randn(T, V, device="cuda").to(torch.bfloat16)
    tg = torch.randint(0, V, (T,), device="cuda")
    cases.append(("cross_entropy fwd+bwd 4096x128256", lambda: ops.cross_entropy_fwd_bwd(logits, tg, inplace_grad=True), 3 * T * V * 2))
    n = 218 * 1024 * 1024
    master, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    pb, g = torch.zeros(n, device="cuda", dtype=torch.bfloat16), torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    cases.append(("adamw_flat 218M params", lambda: ops.adamw_flat_(master, pb, m, v, g, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                                                                    weight_decay=0.1, step=2), n * 28))
    for name, fn, nbytes in cases:
        med, best = time_fn(fn)
        r = {"case": name, "ms_median": med, "gbs": nbytes / med / 1e6, "frac_of_hbm": nbytes / best / 1e6 / pk["hbm_gbs"], "peak_src": pk["src"]}
        results.append(r)
        print(json.dumps(r), flush=True)


def single_gemm():
    """Three launches of one 8192x8192x4096 bf16 GEMM (a small, self-terminating case for profiler captures)."""
    from ferrotorch_b200 import ops
    a = torch.randn(8192, 4096, device="cuda").to(torch.bfloat16)
    b = torch.randn(8192, 4096, device="cuda").to(torch.bfloat16)
    out = torch.empty(8192, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        ops.gemm(a, b, out=out)
    torch.cuda.synchronize()
    print("gemm1 done", float(out[0, 0]))


def single_attn():
    """Three launches of causal attention forward (and backward when built) at B=1 S=4096 Hq=32 Hkv=8."""
    from ferrotorch_b200 import ops
    B, S, Hq, Hkv, D = 1, 4096, 32, 8, 128
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device="cuda").to(torch.bfloat16)
    for _ in range(3):
        out, lse = ops.flash_fwd(qkv, B, S, Hq, Hkv, D, True)
        ops.flash_bwd(qkv, out, lse, torch.ones_like(out), B, S, Hq, Hkv, D, True)
    torch.cuda.synchronize()
    print("attn1 done", float(out[0, 0]))


def single_norm():
    """Three launches each of the RMSNorm forward (with residual) and backward at 16384 x 4096 bf16 (128 MB per tensor, larger than L2): a
    small, self-terminating case for profiler captures."""
    from ferrotorch_b200 import ops
    T, d = 16384, 4096
    x = torch.randn(T, d, device="cuda").to(torch.bfloat16)
    r = torch.randn(T, d, device="cuda").to(torch.bfloat16)
    w = torch.ones(d, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        y, rstd, xs = ops.rmsnorm_fwd(x, w, 1e-5, residual=r)
        dx, dw = ops.rmsnorm_bwd(xs, w, y, rstd)
    torch.cuda.synchronize()
    print("norm1 done", float(y[0, 0]), float(dx[0, 0]))


def single_elementwise():
    """Two launches each of SwiGLU forward / backward (4096 x 14336), rotary embedding, the fused cross-entropy (4096 x 128256) and the flat
    AdamW update (64 M parameters, 1.8 GB of state): every tensor is larger than L2 and the whole case holds about 4 GB, for profiler captures."""
    from ferrotorch_b200 import ops
    T, F, V, n = 4096, 14336, 128256, 64 << 20
    gu = torch.randn(T, 2 * F, device="cuda").to(torch.bfloat16)
    da = torch.randn(T, F, device="cuda").to(torch.bfloat16)
    qkv = torch.randn(T, 48 * 128, device="cuda").to(torch.bfloat16)
    cos, sin = ops.rope_tables(T, 128, 500000.0, "cuda")
    tg = torch.randint(0, V, (T,), device="cuda")
    master, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    pb, g = torch.zeros(n, device="cuda", dtype=torch.bfloat16), torch.full((n,), 0.01, device="cuda", dtype=torch.bfloat16)
    for i in range(2):
        ops.swiglu_fwd(gu)
        ops.swiglu_bwd(gu, da)
        ops.rope_inplace(qkv, cos, sin, T, 0, 40, 128)
        logits = torch.randn(T, V, device="cuda").to(torch.bfloat16)
        loss, _, _ = ops.cross_entropy_fwd_bwd(logits, tg, inplace_grad=True)
        ops.adamw_flat_(master, pb, m, v, g, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=i + 1)
    torch.cuda.synchronize()
    print("ew1 done", float(loss), float(master[0]))


def single_conv_paged():
    """Two launches each of the implicit-GEMM 3x3 convolution (forward and input gradient, 64 x 256 x 56 x 56 channels-last bf16: 103 MB per
    activation tensor) and of the paged decode attention at the per-rank shape of 70B TP=8 (8 query heads, 1 KV head, batch 8, 2304 cached
    tokens): a small, self-terminating case for profiler captures."""
    import math
    from ferrotorch_b200 import _lib, ops
    x = torch.randn(64, 256, 56, 56, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last).requires_grad_()
    w = (torch.randn(256, 256, 3, 3, device="cuda") * 0.02).to(torch.bfloat16)
    Hq, Hkv, B, L, nsplit, D = 8, 1, 8, 2304, 16, 128
    mb = (L + 15) // 16
    kc = torch.randn(B * mb, 16, Hkv, D, device="cuda").to(torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.arange(B * mb, device="cuda", dtype=torch.int32).view(B, mb)
    lens = torch.full((B,), L, device="cuda", dtype=torch.int32)
    q = torch.randn(B, Hq, D, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    ws = torch.zeros(B * Hkv * nsplit * (Hq // Hkv) * 132, device="cuda")
    ctr = torch.zeros(B * Hkv, device="cuda", dtype=torch.int32)
    for _ in range(2):
        y = ops.conv3x3(x, w)
        (gx,) = torch.autograd.grad(y, x, torch.ones_like(y))
        _lib.call("ft_paged_attn_decode", q, kc, vc, bt, mb, lens, B, Hq, Hkv, D, 1 / math.sqrt(D), nsplit, ws, ctr, out, _lib.S())
    torch.cuda.synchronize()
    print("conv1 done", float(y[0, 0, 0, 0]), float(gx[0, 0, 0, 0]), float(out[0, 0, 0]))


PAGED_CASES = [(8, 1, 8, 2304, 16), (8, 1, 8, 2304, 37), (64, 8, 8, 2304, 4), (64, 8, 8, 2304, 16)]
PAGED_SWEEP = [(Hq, Hkv, B, L, n) for Hq, Hkv, B, L in [(8, 1, 8, 2304), (8, 1, 8, 640), (8, 1, 1, 2304), (8, 1, 32, 2304), (64, 8, 8, 2304), (32, 8, 8, 2304)]
               for n in (1, 2, 4, 6, 8, 12, 16, 24, 37, 64)]


def bench_paged(results, cases=PAGED_CASES):
    """Paged decode attention at the per-rank shapes of 70B TP=8 (1 KV head, 8 query heads) and TP=1; `paged_sweep` walks the split
    count at several batch sizes and lengths (the table the decode engine's choice of split count rests on)."""
    import math
    from ferrotorch_b200 import _lib
    pk = peaks()
    for Hq, Hkv, B, L, nsplit in cases:
        D, mb = 128, (L + 15) // 16
        kc = torch.randn(B * mb, 16, Hkv, D, device="cuda").to(torch.bfloat16)
        vc = torch.randn_like(kc)
        bt = torch.arange(B * mb, device="cuda", dtype=torch.int32).view(B, mb)
        lens = torch.full((B,), L, device="cuda", dtype=torch.int32)
        q = torch.randn(B, Hq, D, device="cuda").to(torch.bfloat16)
        out = torch.empty_like(q)
        ws = torch.zeros(B * Hkv * nsplit * (Hq // Hkv) * 132, device="cuda")
        ctr = torch.zeros(B * Hkv, device="cuda", dtype=torch.int32)
        fn = lambda: _lib.call("ft_paged_attn_decode", q, kc, vc, bt, mb, lens, B, Hq, Hkv, D, 1 / math.sqrt(D), nsplit, ws, ctr, out, _lib.S())
        med, best = time_fn(fn, iters=20)
        nbytes = B * L * Hkv * D * 2 * 2
        r = {"case": f"paged_attn_decode B{B} L{L} Hq{Hq} Hkv{Hkv} nsplit{nsplit}", "us_median": med * 1e3, "gbs": nbytes / med / 1e6,
             "frac_of_hbm": nbytes / best / 1e6 / pk["hbm_gbs"]}
        results.append(r)
        print(json.dumps(r), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", nargs="?", default="all")
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    res = []
    if a.what == "gemm1":
        return single_gemm()
    if a.what == "attn1":
        return single_attn()
    if a.what == "norm1":
        return single_norm()
    if a.what == "ew1":
        return single_elementwise()
    if a.what == "conv1":
        return single_conv_paged()
    if a.what in ("gemm", "all"):
        bench_gemm(res)
    if a.what in ("attn", "all"):
        bench_attn(res)
    if a.what == "paged_sweep":
        bench_paged(res, PAGED_SWEEP)
    if a.what in ("paged", "all"):
        bench_paged(res)
    if a.what in ("elementwise", "all"):
        bench_elementwise(res)
    if a.json:
        Path(a.json).parent.mkdir(parents=True, exist_ok=True)
        Path(a.json).write_text(json.dumps({"peaks": peaks(), "results": res}, indent=1))


if __name__ == "__main__":
    main()
