"""Kernel micro-benchmarks: ``python benchmarks/bench_kernels.py [gemm|elementwise|all]``.

Each kernel is timed with CUDA events on the launching stream after warm-up,
with an L2 flush (a write larger than the 126 MB L2) between timed iterations.
For GEMMs the cuBLAS time of the same shape (``torch.matmul``) is printed next
to ours, and both are given as a fraction of the measured peaks in
``MEASURED_PEAKS.json`` when that file is present.
"""
from __future__ import annotations

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from multimesh_jax_b200.ops import kernels as K


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


_flush_buf = None


def flush_l2():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_ms(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def bench_gemm():
    peak, _, how = _peaks()
    T = 8192
    shapes = [
        ("qkv_fwd", T, 12288, 4096), ("attn_out_fwd", T, 4096, 4096), ("gate_up_fwd", T, 22016, 4096),
        ("down_fwd", T, 4096, 11008), ("lm_head_fwd", T, 32000, 4096),
    ]
    rows = []
    for name, M, N, Kd in shapes:
        x = torch.randn(M, Kd, device="cuda").bfloat16()
        w = (torch.randn(N, Kd, device="cuda") * 0.02).bfloat16()
        dy = torch.randn(M, N, device="cuda").bfloat16()
        dw = torch.zeros(N, Kd, device="cuda", dtype=torch.float32)
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(M, Kd, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * M * N * Kd
        for kind, ours, ref in [
            ("fwd", lambda: K.linear_fwd(x, w, out=y), lambda: torch.matmul(x, w.t(), out=y)),
            ("dgrad", lambda: K.linear_dgrad(dy, w, out=dx), lambda: torch.matmul(dy, w, out=dx)),
            ("wgrad", lambda: K.linear_wgrad(dy, x, out=dw, accumulate=True),
             lambda: torch.matmul(dy.t(), x)),
        ]:
            t_ours, t_ref = time_ms(ours), time_ms(ref)
            rows.append({"shape": name, "kind": kind, "M": M, "N": N, "K": Kd,
                         "ours_ms": round(t_ours, 4), "cublas_ms": round(t_ref, 4),
                         "ours_tflops": round(flops / t_ours / 1e9, 1),
                         "cublas_tflops": round(flops / t_ref / 1e9, 1),
                         f"ours_frac_of_{how}_peak": round(flops / t_ours / 1e9 / peak, 3)})
            print(json.dumps(rows[-1]), flush=True)
        del x, w, dy, dw, y, dx
    assert K.read_status() == 0
    return rows


def bench_elementwise():
    _, hbm, how = _peaks()
    T, D, F, V = 8192, 4096, 11008, 32000
    x = torch.randn(T, D, device="cuda").bfloat16()
    w = torch.ones(D, device="cuda").bfloat16()
    gu = torch.randn(T, 2 * F, device="cuda").bfloat16()
    dh = torch.randn(T, F, device="cuda").bfloat16()
    logits = torch.randn(T, V, device="cuda").bfloat16()
    tgt = torch.randint(0, V, (T,), device="cuda")
    y, rstd = K.rmsnorm_fwd(x, w, 1e-5)
    n = 64 << 20
    master, m, v, g = (torch.zeros(n, device="cuda") for _ in range(4))
    p = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    cases = [
        ("rmsnorm_fwd", lambda: K.rmsnorm_fwd(x, w, 1e-5), 2 * T * D * 2),
        ("rmsnorm_bwd", lambda: K.rmsnorm_bwd(x, w, x, rstd), 3 * T * D * 2),
        ("swiglu_fwd", lambda: K.swiglu_fwd(gu), 3 * T * F * 2),
        ("swiglu_bwd", lambda: K.swiglu_bwd(gu, dh), 5 * T * F * 2),
        ("cross_entropy", lambda: K.cross_entropy_fwd_bwd(logits, tgt, 1.0), 3 * T * V * 2),
        ("adamw", lambda: K.adamw_step_(master, p, m, v, g, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                                        weight_decay=0.1, step=1), n * 30),
    ]
    rows = []
    for name, fn, nbytes in cases:
        t = time_ms(fn)
        rows.append({"kernel": name, "ms": round(t, 4), "GBps": round(nbytes / t / 1e6, 1),
                     f"frac_of_{how}_hbm": round(nbytes / t / 1e6 / hbm, 3)})
        print(json.dumps(rows[-1]), flush=True)
    return rows


def main(argv):
    what = argv[1] if len(argv) > 1 else "all"
    if what in ("gemm", "all"):
        bench_gemm()
    if what in ("elementwise", "all"):
        bench_elementwise()


if __name__ == "__main__":
    main(sys.argv)
