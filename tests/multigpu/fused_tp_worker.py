"""Worker of the multi-GPU fused tensor-parallel test (one process per GPU, launched by torchrun)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl")
    from multimesh_jax_b200.ops import kernels as K
    from multimesh_jax_b200.parallel import symm
    from multimesh_jax_b200.parallel.tp import FusedLinearAllReduce

    arena = symm.SymmetricArena(512 << 20, dev)
    op = FusedLinearAllReduce(arena, list(range(world)))
    ok = True
    # 384 and 640 rows: an odd number of 128-row blocks, so the second CTA of the last pair has no rows
    for it, (M, N, Kd, b_mn) in enumerate([(1024, 4096, 1024, False), (1024, 4096, 1024, False), (8192, 4096, 2048, False),
                                           (1024, 4096, 1024, True), (384, 512, 320, False), (8192, 4096, 2048, True),
                                           (640, 768, 256, False), (8192, 4096, 2048, False)]):
        torch.manual_seed(100 * it + rank)
        a = torch.randn(M, Kd, device=dev).bfloat16()
        b = (torch.randn(Kd, N, device=dev) if b_mn else torch.randn(N, Kd, device=dev)).bfloat16()
        out = op(a, b, b_mn=b_mn)
        ref = a.float() @ (b.float() if b_mn else b.float().t())
        dist.all_reduce(ref)
        torch.cuda.synchronize()
        err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
        if err > 2e-2:
            ok = False
            print(f"rank {rank}: case {it} relative error {err}", flush=True)
    # GEMM fused with its reduce-scatter: rows owned in `outer` chunks per rank (a [B, S, .] product
    # scattered on S has one chunk per sequence)
    from multimesh_jax_b200.parallel.tp import FusedLinearReduceScatter
    rs = FusedLinearReduceScatter(arena, list(range(world)))
    for it, (M, N, Kd, b_mn, outer) in enumerate([(1024, 1024, 512, False, 1), (1024, 1024, 512, False, 1),
                                                  (8192, 4096, 2048, False, 4), (2048, 768, 320, True, 2),
                                                  (8192, 4096, 2048, False, 4), (world * 128, 512, 256, False, 1),
                                                  (8192, 4096, 6144, True, 4)]):
        assert rs.supported(M, N, Kd, outer, torch.bfloat16)
        torch.manual_seed(500 * it + rank)
        a = torch.randn(M, Kd, device=dev).bfloat16()
        b = (torch.randn(Kd, N, device=dev) if b_mn else torch.randn(N, Kd, device=dev)).bfloat16()
        out = rs(a, b, b_mn=b_mn, outer=outer)
        ref = a.float() @ (b.float() if b_mn else b.float().t())
        dist.all_reduce(ref)
        mine = ref.view(outer, world, M // (outer * world), N)[:, rank].reshape(M // world, N)
        torch.cuda.synchronize()
        err = (out.float() - mine).norm().item() / mine.norm().item()
        worst = (out.float() - mine).abs().max().item() / mine.abs().max().item()
        if err > 1e-2 or worst > 2e-2:
            ok = False
            print(f"rank {rank}: reduce-scatter case {it}: relative Frobenius error {err}, max {worst}", flush=True)
    # all-gather fused into the GEMM: every rank holds a row shard of the activations
    from multimesh_jax_b200.parallel.tp import FusedAllGatherLinear
    ag = FusedAllGatherLinear(arena, list(range(world)))
    for it, (Ms, N, Kd, b_mn, outer) in enumerate([(512, 1024, 512, False, 1), (512, 1024, 512, False, 1),
                                                   (4096, 6144, 4096, False, 4), (1024, 768, 2048, True, 2),
                                                   (4096, 6144, 4096, False, 4), (384, 512, 256, False, 3),
                                                   (128, 512, 256, False, 1)]):
        assert ag.supported(Ms, Kd, outer, torch.bfloat16)
        torch.manual_seed(1000 + 10 * it + rank)
        a = torch.randn(Ms, Kd, device=dev).bfloat16()
        torch.manual_seed(2000 + it)
        b = (torch.randn(Kd, N, device=dev) if b_mn else torch.randn(N, Kd, device=dev)).bfloat16()
        out, a_full = ag(a, b, b_mn=b_mn, outer=outer)
        parts = [torch.empty_like(a) for _ in range(world)]
        dist.all_gather(parts, a)
        # chunk c of the gathered rows is chunk c // world of rank c % world
        ref_a = torch.stack([p.view(outer, Ms // outer, Kd) for p in parts], dim=1).reshape(world * Ms, Kd)
        ref = ref_a.float() @ (b.float() if b_mn else b.float().t())
        torch.cuda.synchronize()
        if not torch.equal(a_full, ref_a):
            ok = False
            print(f"rank {rank}: all-gather case {it}: gathered rows differ", flush=True)
        err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
        if err > 2e-2:
            ok = False
            print(f"rank {rank}: all-gather case {it} relative error {err}", flush=True)
    status = K.read_status()
    if status != 0:
        ok = False
        print(f"rank {rank}: kernel status {status}", flush=True)
    t = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("FUSED_TP_OK" if t.item() == 1 else "FUSED_TP_FAILED", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
