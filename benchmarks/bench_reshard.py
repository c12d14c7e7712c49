"""Cross-submesh reshard micro-benchmark.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        benchmarks/bench_reshard.py [--max-mb 4096] [--pairs 1-1,2-2]

Tensors are bf16 ``[B, S, 8192]`` of N(0,1) values from 1 MB to 4 GB in powers of 4. For a
pair ``M-N`` the source submesh is ranks ``[0, M)`` and the destination submesh ranks
``[M, M+N)`` (needs ``W >= M+N``). Transitions: batch->hidden (all-to-all pattern),
hidden->replicated (all-gather pattern) and replicated->batch (slice of one replica).

For each case two implementations are timed on the device (CUDA events on the destination
ranks, max over ranks, after warm-up):
  * ``pull`` - the hand-written kernel reading source tiles directly from peer HBM,
  * ``nccl`` - point-to-point messages (``batch_isend_irecv``), the baseline,
and compared with the NVLink roofline: the largest number of bytes any GPU must receive or
send, divided by the measured 770 GB/s per direction (or the HBM copy bandwidth for purely
local moves). One JSON line per case is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def shapes_for(total_bytes: int):
    hidden = 8192
    B = 8
    S = max(1, total_bytes // (B * hidden * 2))
    return [B, S, hidden]


def make_shape(_mm_C, sizes, kind: str, start: int, n: int):
    if kind == "batch":
        return _mm_C.sharded_shape("bfloat16", sizes, [[0], [], []], [n], start)
    if kind == "hidden":
        return _mm_C.sharded_shape("bfloat16", sizes, [[], [], [0]], [n], start)
    return _mm_C.sharded_shape("bfloat16", sizes, [[], [], []], [n], start)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=4096)
    ap.add_argument("--min-mb", type=int, default=1)
    ap.add_argument("--pairs", default="")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--check", action="store_true", help="verify the moved data against the source values")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl")
    from .. import _mm_C
    from ..runtime.collectives import Topology
    from . import symm
    from .reshard import run_reshard_dist

    topo = Topology("dist", world, rank=rank, device=dev)
    pairs = [(1, 1), (2, 2), (4, 4), (4, 2), (2, 4)]
    if args.pairs:
        pairs = [tuple(int(x) for x in p.split("-")) for p in args.pairs.split(",")]
    pairs = [(m, n) for m, n in pairs if m + n <= world]
    sizes_mb = [s for s in (1, 4, 16, 64, 256, 1024, 4096) if args.min_mb <= s <= args.max_mb]
    max_bytes = max(sizes_mb) << 20
    arena = symm.SymmetricArena(2 * max_bytes + (64 << 20), dev)
    transitions = [("batch", "hidden"), ("hidden", "replicated"), ("replicated", "batch")]

    for m, n in pairs:
        for src_kind, dst_kind in transitions:
            for mb in sizes_mb:
                sizes = shapes_for(mb << 20)
                total_bytes = sizes[0] * sizes[1] * sizes[2] * 2
                src = make_shape(_mm_C, sizes, src_kind, 0, m)
                dst = make_shape(_mm_C, sizes, dst_kind, m, n)
                plan = _mm_C.plan_reshard(src, dst)
                arena.reset()
                src_t = arena.alloc(src["shard_size"], torch.bfloat16)
                dst_t = arena.alloc(dst["shard_size"], torch.bfloat16)
                is_src, is_dst = rank < m, m <= rank < m + n
                if is_src:
                    # value = f(global index) so that the check does not need the whole tensor
                    lo, hi = _mm_C.tile_box(src, rank)
                    g = torch.Generator(device=dev).manual_seed(1000 + lo[0] * 7 + lo[2])
                    src_t.local.copy_(torch.randn(src["shard_size"], generator=g, device=dev, dtype=torch.float32))
                arena.barrier()
                mine = [c for c in plan["chunks"] if c["dst_device"] == rank]
                mine_src = [c for c in plan["chunks"] if c["src_device"] == rank]
                records = symm.build_pull_chunks(mine, src["shard_size"], dst["shard_size"], src_t.ptr,
                                                 dst_t.ptr(rank), 2) if mine else []

                def run_pull():
                    if records:
                        symm.reshard_pull(records, 2, arena)

                def run_nccl():
                    out, _ = run_reshard_dist(topo, rank, src_t.local if is_src else None, mine_src, mine, dst)
                    return out

                results = {}
                for name, fn in (("pull", run_pull), ("nccl", run_nccl)):
                    for _ in range(2):
                        fn()
                    arena.barrier()
                    times = []
                    for _ in range(args.iters):
                        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        dist.barrier()
                        s.record()
                        fn()
                        e.record()
                        torch.cuda.synchronize()
                        times.append(s.elapsed_time(e))
                    t = torch.tensor([sorted(times)[len(times) // 2] if (is_dst or name == "nccl") else 0.0], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    results[name] = float(t.item())
                ok = True
                if args.check:
                    # compare the pulled tile with the NCCL result (every rank takes part in the exchange)
                    ref = run_nccl()
                    if is_dst and mine:
                        ok = bool(torch.equal(ref, dst_t.local))
                okt = torch.tensor([1 if ok else 0], device=dev)
                dist.all_reduce(okt, op=dist.ReduceOp.MIN)
                # roofline: busiest link direction
                ingress = {}
                egress = {}
                for c in plan["chunks"]:
                    vol = 2
                    for a, b in zip(c["lo"], c["hi"]):
                        vol *= (b - a)
                    if c["src_device"] != c["dst_device"]:
                        ingress[c["dst_device"]] = ingress.get(c["dst_device"], 0) + vol
                        egress[c["src_device"]] = egress.get(c["src_device"], 0) + vol
                busiest = max(list(ingress.values()) + list(egress.values()) + [0])
                roof_ms = busiest / (LINK_GBS * 1e9) * 1e3
                moved = sum(ingress.values())
                if rank == 0:
                    row = {"pair": f"{m}->{n}", "transition": f"{src_kind}->{dst_kind}", "tensor_mb": mb,
                           "bytes_over_links": moved, "pull_ms": round(results["pull"], 4),
                           "nccl_ms": round(results["nccl"], 4),
                           "pull_GBps": round(moved / results["pull"] / 1e6, 1) if results["pull"] > 0 else None,
                           "nccl_GBps": round(moved / results["nccl"] / 1e6, 1) if results["nccl"] > 0 else None,
                           "roofline_ms": round(roof_ms, 4),
                           "pull_frac_of_roofline": round(roof_ms / results["pull"], 3) if results["pull"] > 0 else None,
                           "check": bool(okt.item())}
                    print(json.dumps(row), flush=True)
    from ..ops import kernels as K
    status = K.read_status()
    if rank == 0:
        print(json.dumps({"kernel_status": status}))
    arena.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
