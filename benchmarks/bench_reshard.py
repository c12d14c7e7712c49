"""Cross-submesh reshard micro-benchmark.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 \
        benchmarks/bench_reshard.py [--max-mb 4096] [--min-mb 1] [--pairs 1-1,2-2,4-4,4-2,2-4] [--check]

Tensors are bf16 ``[B, S, 8192]`` of N(0,1) values from 1 MB to 4 GB in powers of 4. For a
pair ``M-N`` the source submesh is ranks ``[0, M)`` and the destination submesh ranks
``[M, M+N)`` (needs ``W >= M+N``). Transitions: batch->hidden (all-to-all pattern),
hidden->replicated (all-gather pattern) and replicated->batch (slice of one replica).

First the peer link is probed in the same run: a plain 16-byte copy kernel pulls 1 GiB from a
peer's memory, once with a single GPU pulling (``probe_single_gbs``) and once with every GPU
pulling from its ring neighbour at the same time (``probe_all_gbs``). Then, for each case, two
implementations are timed on the device (CUDA events, median of the iterations, max over
ranks, after warm-up):
  * ``pull`` - the protocol the training step runs: the source ranks raise their ready flags,
    every destination rank's pull kernel waits for the flags of its sources, reads the source
    tiles straight from peer HBM, writes its own layout and raises the done flags. The source
    tile is where the producer left it: nothing is staged.
  * ``nccl`` - point-to-point messages (``batch_isend_irecv``), the baseline.
The roofline of a case is the largest number of bytes any GPU must receive or send divided by
a link rate; the fraction is reported against the probed single-puller rate and against the
nominal 900 GB/s per direction. One JSON line per case is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

NOMINAL_GBS = 900.0


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


def _median_ms(fn, iters, sync):
    times = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return sorted(times)[len(times) // 2]


def probe_link(arena, lib, rank, world, dev, nbytes):
    """GB/s of a plain copy kernel reading a peer's memory: one puller, then all at once."""
    from multimesh_jax_b200.ops import _lib
    src = arena.alloc([nbytes // 2], torch.bfloat16)
    dst = torch.empty(nbytes // 2, dtype=torch.bfloat16, device=dev)
    src.peer(rank).normal_()
    arena.barrier()
    stream = lambda: torch.cuda.current_stream().cuda_stream
    peer = (rank + 1) % world

    def pull():
        _lib.check(lib.mm_peer_copy(dst.data_ptr(), src.ptr(peer), nbytes, stream()), "mm_peer_copy")

    def local():
        _lib.check(lib.mm_peer_copy(dst.data_ptr(), src.ptr(rank), nbytes, stream()), "mm_peer_copy")
    out = {}
    for name, fn, active in (("probe_single_gbs", pull, rank == 0), ("probe_all_gbs", pull, True), ("local_copy_gbs", local, True)):
        for _ in range(2):
            if active:
                fn()
        torch.cuda.synchronize()
        ms = _median_ms(fn if active else (lambda: None), 5, dist.barrier)
        t = torch.tensor([ms if active else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = round(nbytes / float(t.item()) / 1e6, 1)
    ok = bool(torch.equal(dst, src.peer(rank))) if world == 1 else True
    out["probe_bytes"] = nbytes
    out["probe_copy_intact"] = ok
    arena.barrier()
    return out


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
    from multimesh_jax_b200 import _mm_C
    from multimesh_jax_b200.ops import kernels as K
    from multimesh_jax_b200.parallel import symm
    from multimesh_jax_b200.parallel.reshard import run_reshard_dist
    from multimesh_jax_b200.runtime.collectives import Topology

    topo = Topology("dist", world, rank=rank, device=dev)
    pairs = [(1, 1), (2, 2), (4, 4), (4, 2), (2, 4)]
    if args.pairs:
        pairs = [tuple(int(x) for x in p.split("-")) for p in args.pairs.split(",")]
    pairs = [(m, n) for m, n in pairs if m + n <= world]
    sizes_mb = [s for s in (1, 4, 16, 64, 256, 1024, 4096) if args.min_mb <= s <= args.max_mb]
    max_bytes = max(sizes_mb) << 20
    arena = symm.SymmetricArena(2 * max_bytes + (64 << 20), dev)
    counter = arena.alloc_counter("bench_reshard")
    # flags: one ready word per source rank and one done word per destination rank, reused by every case
    ready = [arena.alloc_flag() for _ in range(world)]
    done = [arena.alloc_flag() for _ in range(world)]
    epoch = 0

    probe = probe_link(arena, arena.lib, rank, world, dev, min(1 << 30, max_bytes))
    if rank == 0:
        print(json.dumps(probe), flush=True)
    link = probe["probe_single_gbs"]
    transitions = [("batch", "hidden"), ("hidden", "replicated"), ("replicated", "batch")]

    for m, n in pairs:
        for src_kind, dst_kind in transitions:
            for mb in sizes_mb:
                sizes = shapes_for(mb << 20)
                src = make_shape(_mm_C, sizes, src_kind, 0, m)
                dst = make_shape(_mm_C, sizes, dst_kind, m, n)
                plan = _mm_C.plan_reshard(src, dst)
                arena.reset()
                src_t = arena.alloc(src["shard_size"], torch.bfloat16)
                dst_t = arena.alloc(dst["shard_size"], torch.bfloat16)
                is_src, is_dst = rank < m, m <= rank < m + n
                if is_src:
                    lo, hi = _mm_C.tile_box(src, rank)
                    g = torch.Generator(device=dev).manual_seed(1000 + lo[0] * 7 + lo[2])
                    src_t.peer(rank).copy_(torch.randn(src["shard_size"], generator=g, device=dev, dtype=torch.float32))
                arena.barrier()
                mine = [c for c in plan["chunks"] if c["dst_device"] == rank]
                mine_src = [c for c in plan["chunks"] if c["src_device"] == rank]
                records = symm.build_pull_chunks(mine, src["shard_size"], dst["shard_size"], src_t.ptr,
                                                 dst_t.ptr(rank), 2) if mine else []
                readers = sorted({c["dst_device"] for c in mine_src})
                writers = sorted({c["src_device"] for c in mine})

                def run_pull():
                    nonlocal epoch
                    epoch += 1
                    if mine_src:
                        symm.set_flags(arena, [arena.flag_ptr(r, ready[rank]) for r in readers], epoch)
                    if records:
                        waits = [arena.flag_ptr(rank, ready[w]) for w in writers]
                        dones = [arena.flag_ptr(w, done[rank]) for w in writers]
                        for i in range(0, len(records), 64):
                            last = i + 64 >= len(records)
                            symm.reshard_pull(records[i:i + 64], 2, arena, wait_flags=waits if i == 0 else (),
                                              wait_value=epoch, done_flags=dones if last else (), done_value=epoch,
                                              counter=counter)
                    if mine_src:      # the tile may be overwritten only after its readers are done
                        symm.wait_flags(arena, [arena.flag_ptr(rank, done[r]) for r in readers], epoch)

                def run_nccl():
                    out, _ = run_reshard_dist(topo, rank, src_t.peer(rank) if is_src else None, mine_src, mine, dst)
                    return out

                results = {}
                for name, fn in (("pull", run_pull), ("nccl", run_nccl)):
                    for _ in range(2):
                        fn()
                    arena.barrier()
                    ms = _median_ms(fn, args.iters, dist.barrier)
                    t = torch.tensor([ms], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    results[name] = float(t.item())
                ok = True
                if args.check:
                    # compare the pulled tile with the NCCL result (every rank takes part in the exchange)
                    ref = run_nccl()
                    if is_dst and mine:
                        ok = bool(torch.equal(ref, dst_t.peer(rank)))
                okt = torch.tensor([1 if ok else 0], device=dev)
                dist.all_reduce(okt, op=dist.ReduceOp.MIN)
                # roofline: busiest link direction
                ingress, egress = {}, {}
                for c in plan["chunks"]:
                    vol = 2
                    for a, b in zip(c["lo"], c["hi"]):
                        vol *= (b - a)
                    if c["src_device"] != c["dst_device"]:
                        ingress[c["dst_device"]] = ingress.get(c["dst_device"], 0) + vol
                        egress[c["src_device"]] = egress.get(c["src_device"], 0) + vol
                busiest = max(list(ingress.values()) + list(egress.values()) + [0])
                moved = sum(ingress.values())
                if rank == 0:
                    pull_ms, nccl_ms = results["pull"], results["nccl"]
                    row = {"pair": f"{m}->{n}", "transition": f"{src_kind}->{dst_kind}", "tensor_mb": mb,
                           "bytes_over_links": moved, "busiest_direction_bytes": busiest,
                           "pull_ms": round(pull_ms, 4), "nccl_ms": round(nccl_ms, 4),
                           "pull_GBps_per_busiest_gpu": round(busiest / pull_ms / 1e6, 1) if pull_ms > 0 else None,
                           "nccl_GBps_per_busiest_gpu": round(busiest / nccl_ms / 1e6, 1) if nccl_ms > 0 else None,
                           "pull_frac_of_probed": round(busiest / (link * 1e6) / pull_ms, 3) if pull_ms > 0 else None,
                           "pull_frac_of_900": round(busiest / (NOMINAL_GBS * 1e6) / pull_ms, 3) if pull_ms > 0 else None,
                           "nccl_frac_of_probed": round(busiest / (link * 1e6) / nccl_ms, 3) if nccl_ms > 0 else None,
                           "check": bool(okt.item())}
                    print(json.dumps(row), flush=True)
    status = K.read_status()
    if rank == 0:
        print(json.dumps({"kernel_status": status}))
    arena.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
