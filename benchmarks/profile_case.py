"""One kernel, one small case, three launches - the program to put under a profiler.

    python benchmarks/profile_case.py gemm|gemm_dgrad|gemm_wgrad (each also as <case>_pair)|gemm_allreduce_loopback|gemm_reducescatter_loopback|gemm_allgather_loopback|reshard_pull_local|moe_dispatch_local|flash_fwd|flash_bwd|rmsnorm_bwd|swiglu|adamw|cross_entropy

Inputs are larger than the 126 MB L2 where the kernel is memory bound and a few hundred MB at
most, so a full-metric capture of one launch finishes in seconds. Each case prints its
CUDA-event time (after one warm-up launch) and the algorithmic FLOPs / bytes, so that the
numbers in a profile can be checked against an unprofiled run of the same command.
"""
from __future__ import annotations

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from multimesh_jax_b200.ops import attention
from multimesh_jax_b200.ops import kernels as K


def _time(fn, launches=2):
    fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(launches):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / launches


def main(argv=None) -> int:
    case = (argv or sys.argv[1:] or ["gemm"])[0]
    dev = torch.device("cuda")
    torch.manual_seed(0)
    out = {"case": case}
    if case.endswith("_pair"):     # same case on the CTA-pair kernel
        K.PAIR_MIN_M = 1
        case = case[:-5]
    if case in ("gemm", "gemm_dgrad", "gemm_wgrad"):
        M, N, Kd = 8192, 4096, 4096
        if case == "gemm":          # y = x w^T
            a = torch.randn(M, Kd, device=dev).bfloat16()
            b = torch.randn(N, Kd, device=dev).bfloat16()
            fn = lambda: K.linear_fwd(a, b)
        elif case == "gemm_dgrad":  # dx = dy w
            a = torch.randn(M, N, device=dev).bfloat16()
            b = torch.randn(N, Kd, device=dev).bfloat16()
            fn = lambda: K.linear_dgrad(a, b)
        else:                       # dw += dy^T x, fp32 accumulator
            a = torch.randn(M, N, device=dev).bfloat16()
            b = torch.randn(M, Kd, device=dev).bfloat16()
            acc = torch.zeros(N, Kd, device=dev, dtype=torch.float32)
            fn = lambda: K.linear_wgrad(a, b, out=acc, accumulate=True)
        ms = _time(fn)
        out.update(shape=[M, N, Kd], ms=ms, tflops=2.0 * M * N * Kd / ms / 1e9)
    elif case == "gemm_allreduce_loopback":
        # The fused GEMM + all-reduce kernel on ONE GPU: its single peer slot is this GPU's own
        # receive buffer and flag array, so every tile is pushed to local memory, flagged, waited
        # for and added back (out = 2 A B^T). Same kernel and instruction stream as the 2-GPU call
        # with NVLink replaced by local HBM; no launch waits on another launch.
        from ctypes import c_int64
        from multimesh_jax_b200.parallel import tp  # noqa: F401 - registers the entry point's signature
        from multimesh_jax_b200.ops import _lib
        M, N, Kd = 8192, 4096, 2048
        a = torch.randn(M, Kd, device=dev).bfloat16()
        b = torch.randn(N, Kd, device=dev).bfloat16()
        tiles = 4 * ((M + 127) // 128) * ((N + 255) // 256)
        recv = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
        flags = torch.zeros(tiles, device=dev, dtype=torch.int32)
        res = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        epoch = [0]
        lib = _lib.load()

        def fn():
            epoch[0] += 1
            one = lambda t: (c_int64 * 1)(t.data_ptr())
            rc = lib.mm_gemm_allreduce_bf16(a.data_ptr(), 0, a.stride(0), b.data_ptr(), 0, b.stride(0), res.data_ptr(),
                                            res.stride(0), M, N, Kd, one(recv), one(recv), one(flags), one(flags), 1,
                                            epoch[0], torch.cuda.current_stream().cuda_stream)
            _lib.check(rc, "mm_gemm_allreduce_bf16")
        ms = _time(fn)
        ref = 2.0 * (a.float() @ b.float().t())
        err = float((res.float() - ref).abs().max() / ref.abs().max())
        out.update(shape=[M, N, Kd], ms=ms, tflops=2.0 * M * N * Kd / ms / 1e9, max_rel_err=err,
                   bytes_pushed=M * N * 2)
    elif case == "gemm_reducescatter_loopback":
        # The fused GEMM + reduce-scatter kernel on ONE GPU as rank 0 of 2 with 128-row chunks: the
        # tiles of "rank 1's" rows are pushed into this GPU's own receive slot, whose flags are the
        # ones the reduction of the neighbouring own tile waits for, so every push, flag, wait and
        # add of the 2-GPU call runs with NVLink replaced by local HBM (own row block 2j of the
        # result = rows 2j + rows 2j+1 of A B^T). The two tiles belong to the two CTAs of one pair,
        # which run together: no launch waits on another launch.
        from ctypes import c_int64
        from multimesh_jax_b200.parallel import tp  # noqa: F401
        from multimesh_jax_b200.ops import _lib
        M, N, Kd = 8192, 4096, 2048
        a = torch.randn(M, Kd, device=dev).bfloat16()
        b = torch.randn(N, Kd, device=dev).bfloat16()
        Ms = M // 2
        tiles = 4 * (Ms // 128) * ((N + 255) // 256)
        recv = torch.zeros(Ms, N, device=dev, dtype=torch.bfloat16)
        flags = torch.zeros(tiles, device=dev, dtype=torch.int32)
        res = torch.empty(Ms, N, device=dev, dtype=torch.bfloat16)
        epoch = [0]
        lib = _lib.load()

        def fn():
            epoch[0] += 1
            one = lambda t: (c_int64 * 1)(t.data_ptr())
            two = lambda t: (c_int64 * 2)(0, t.data_ptr())
            rc = lib.mm_gemm_reducescatter_bf16(a.data_ptr(), 0, a.stride(0), b.data_ptr(), 0, b.stride(0), res.data_ptr(),
                                                res.stride(0), M, N, Kd, one(recv), two(recv), one(flags), two(flags), 2, 0,
                                                128, epoch[0], torch.cuda.current_stream().cuda_stream)
            _lib.check(rc, "mm_gemm_reducescatter_bf16")
        ms = _time(fn)
        full = (a.float() @ b.float().t()).view(M // 256, 2, 128, N)
        ref = (full[:, 0] + full[:, 1]).reshape(Ms, N)
        err = float((res.float() - ref).abs().max() / ref.abs().max())
        out.update(shape=[M, N, Kd], ms=ms, tflops=2.0 * M * N * Kd / ms / 1e9, max_rel_err=err,
                   bytes_pushed=Ms * N * 2)
    elif case == "gemm_allgather_loopback":
        # The fused all-gather + GEMM kernel on ONE GPU as rank 0 of 2: the "peer" shard is a second
        # buffer in local memory, pulled by the helper warps exactly as a peer's would be.
        import ctypes
        from ctypes import c_int64
        from multimesh_jax_b200.parallel import tp  # noqa: F401
        from multimesh_jax_b200.ops import _lib
        Ms, N, Kd = 4096, 6144, 4096
        M = 2 * Ms
        a0 = torch.randn(Ms, Kd, device=dev).bfloat16()
        a1 = torch.randn(Ms, Kd, device=dev).bfloat16()
        b = torch.randn(N, Kd, device=dev).bfloat16()
        gathered = torch.empty(M, Kd, device=dev, dtype=torch.bfloat16)
        ready = torch.zeros(M // 128, device=dev, dtype=torch.int32)
        res = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        target = ctypes.c_int(0)
        lib = _lib.load()

        def fn():
            srcs = (c_int64 * 2)(a0.data_ptr(), a1.data_ptr())
            rc = lib.mm_allgather_gemm_bf16(srcs, 2, 0, gathered.data_ptr(), ready.data_ptr(), ctypes.byref(target),
                                            b.data_ptr(), 0, b.stride(0), res.data_ptr(), res.stride(0), M, N, Kd, 0,
                                            None, 0, None, torch.cuda.current_stream().cuda_stream)
            _lib.check(rc, "mm_allgather_gemm_bf16")
        ms = _time(fn)
        ref = torch.cat([a0, a1]).float() @ b.float().t()
        err = float((res.float() - ref).abs().max() / ref.abs().max())
        out.update(shape=[M, N, Kd], ms=ms, tflops=2.0 * M * N * Kd / ms / 1e9, max_rel_err=err,
                   gathered_ok=bool(torch.equal(gathered, torch.cat([a0, a1]))), bytes_pulled=Ms * Kd * 2)
    elif case == "reshard_pull_local":
        # The reshard pull kernel on ONE GPU: a batch-sharded [8, S, 8192] source (two "devices" =
        # two local buffers) pulled into one hidden-sharded destination tile - 8 KB row pieces from
        # two sources, the all-to-all pattern of a layout-changing stage boundary.
        from multimesh_jax_b200 import _mm_C
        from multimesh_jax_b200.parallel import symm
        B_, S_, H_ = 8, 2048, 8192
        src = _mm_C.sharded_shape("bfloat16", [B_, S_, H_], [[0], [], []], [2], 0)
        dst = _mm_C.sharded_shape("bfloat16", [B_, S_, H_], [[], [], [0]], [2], 0)
        plan = _mm_C.plan_reshard(src, dst)
        tiles = [torch.randn(src["shard_size"], device=dev).bfloat16() for _ in range(2)]
        dtile = torch.empty(dst["shard_size"], device=dev, dtype=torch.bfloat16)
        mine = [c for c in plan["chunks"] if c["dst_device"] == 0]
        recs = symm.build_pull_chunks(mine, list(src["shard_size"]), list(dst["shard_size"]),
                                      lambda d_: tiles[d_].data_ptr(), dtile.data_ptr(), 2)
        arena = symm.SymmetricArena(1 << 20, dev)
        ms = _time(lambda: symm.reshard_pull(recs, 2, arena))
        ref = torch.cat(tiles, dim=0)[:, :, :H_ // 2]
        out.update(shape=[B_, S_, H_], ms=ms, gbs=2.0 * dtile.numel() * 2 / ms / 1e6, ok=bool(torch.equal(dtile, ref)),
                   records=len(recs))
    elif case == "moe_dispatch_local":
        # Router + dispatch kernel on ONE GPU (all 8 experts local): logits, top-2, gates, slot
        # counters and the scatter of every token row into its experts' receive regions.
        from multimesh_jax_b200.parallel import symm
        from multimesh_jax_b200.parallel.ep import PeerMoE
        T, D, E, k = 16384, 4096, 8, 2
        x = (torch.randn(T, D, device=dev) * 0.5).bfloat16()
        wr = (torch.randn(E, D, device=dev) * 0.02).bfloat16()
        arena = symm.SymmetricArena(PeerMoE.required_bytes(T, D, E) + (8 << 20), dev)
        pm = PeerMoE(arena, [arena.rank], T, D, E)
        pm.k = k

        def fn():
            pm.counter.peer(arena.rank).zero_()
            pm._route_dispatch(x, wr, None)
        ms = _time(fn)
        out.update(shape=[T, D, E, k], ms=ms, gbs=(T * D * 2 * (1 + k)) / ms / 1e6)
    elif case in ("flash_fwd", "flash_bwd"):
        B, S, H, D = 2, 2048, 16, 128
        extra = (argv or sys.argv[1:])[1:]
        if len(extra) >= 2:          # flash_fwd / flash_bwd <batch> <heads>: the training step's shape is 4 32
            B, H = int(extra[0]), int(extra[1])
        qkv = (torch.randn(B, S, 3 * H, D, device=dev) * 0.5).bfloat16()
        o, lse = attention.attention_fwd_packed(qkv, 1)
        if case == "flash_fwd":
            ms = _time(lambda: attention.attention_fwd_packed(qkv, 1))
            flops = 4.0 * B * H * S * S * D / 2
        else:
            do = torch.randn_like(o)
            ms = _time(lambda: attention.attention_bwd_packed(do, qkv, o, lse, 1))
            flops = 10.0 * B * H * S * S * D / 2
        out.update(shape=[B, S, H, D], ms=ms, tflops=flops / ms / 1e9)
    elif case == "rmsnorm_bwd":
        T, D = 32768, 4096
        x = torch.randn(T, D, device=dev).bfloat16()
        w = torch.ones(D, device=dev).bfloat16()
        dy = torch.randn(T, D, device=dev).bfloat16()
        _, rstd = K.rmsnorm_fwd(x, w, 1e-5)
        ms = _time(lambda: K.rmsnorm_bwd(x, w, dy, rstd))
        out.update(shape=[T, D], ms=ms, gbs=3.0 * T * D * 2 / ms / 1e6)
    elif case == "swiglu":
        T, F = 16384, 11008
        gu = torch.randn(T, 2 * F, device=dev).bfloat16()
        ms = _time(lambda: K.swiglu_fwd(gu))
        out.update(shape=[T, F], ms=ms, gbs=3.0 * T * F * 2 / ms / 1e6)
    elif case == "adamw":
        n = 64 << 20
        master = torch.randn(n, device=dev)
        p = master.bfloat16()
        m, v, g = torch.zeros_like(master), torch.zeros_like(master), torch.randn(n, device=dev)
        step = torch.ones(1, dtype=torch.int64, device=dev)
        ms = _time(lambda: K.adamw_step_(master, p, m, v, g, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                                         step=step))
        out.update(shape=[n], ms=ms, gbs=n * (4 * 4 + 3 * 4 + 2) / ms / 1e6)
    elif case == "cross_entropy":
        T, V = 8192, 32000
        logits = torch.randn(T, V, device=dev).bfloat16()
        tgt = torch.randint(0, V, (T,), device=dev)
        ms = _time(lambda: K.cross_entropy_fwd_bwd(logits.clone(), tgt, 1.0 / T))
        out.update(shape=[T, V], ms=ms)
    else:
        raise SystemExit(f"unknown case {case}")
    out["kernel_status"] = K.read_status()
    print(json.dumps(out), flush=True)
    # a recorded expiry of a bounded wait or a wrong result fails the run, so that a profiler
    # capture chained behind it with && never replays a kernel that does not finish cleanly
    bad = out["kernel_status"] != 0 or out.get("ok") is False or out.get("gathered_ok") is False \
        or out.get("max_rel_err", 0.0) > 2e-2
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
