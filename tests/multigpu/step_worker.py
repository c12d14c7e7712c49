"""Worker of the multi-GPU training-step tests (one process per GPU, launched by torchrun):
the compiled step on `pp x dp x tp` GPUs against the eager step on one GPU, in bf16.

    step_worker.py <pp> <dp> <tp> [fsdp|moe|sp]      (sp: sequence-parallel tensor parallelism with a vocabulary-sharded loss)
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    pp, dp, tp = (int(a) for a in sys.argv[1:4])
    fsdp = len(sys.argv) > 4 and sys.argv[4] == "fsdp"
    moe = len(sys.argv) > 4 and sys.argv[4] == "moe"
    sp = len(sys.argv) > 4 and sys.argv[4] == "sp"
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl")
    import multimesh_jax_b200 as mm
    from multimesh_jax_b200.models import llama
    from multimesh_jax_b200.ops import kernels as K
    from multimesh_jax_b200.runtime.collectives import tile_box
    from torch.utils import _pytree as pytree

    torch.manual_seed(0)
    cfg = llama.LlamaConfig.tiny(n_layers=2 * pp, d_model=512, n_heads=4, n_kv_heads=2, d_ff=1024, vocab=1024,
                                 n_experts=4 if moe else 0, top_k=2)
    cfg.sequence_parallel = cfg.vocab_parallel = sp
    B, S, MB = 8, 256, 2
    params = llama.init_params(cfg, device="cpu")
    params = pytree.tree_map(lambda t: t.to(dev), params)
    state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S)).to(dev)
    labels = torch.randint(0, cfg.vocab, (B, S)).to(dev)
    cos, sin = llama.rope_tables(cfg, S, dev)
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-3), seq_len=S, global_batch=B, microbatch_size=MB,
                                 fsdp=fsdp)
    mesh = mm.MultiMesh((pp, dp, tp), ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=pp)
    with mesh:
        exe = mm.compile_function(step, (params, state, tokens, labels, cos, sin), mesh=mesh, backend="dist")
    clone = lambda tree: pytree.tree_map(lambda t: t.clone(), tree)
    with mm.ignore_transforms():
        loss_ref, p_ref, s_ref = step(clone(params), clone(state), tokens, labels, cos, sin)
        loss_ref2, p_ref2, _ = step(p_ref, s_ref, tokens, labels, cos, sin)
    loss, p_mm, s_mm = exe(clone(params), clone(state), tokens, labels, cos, sin)
    loss2, p_mm2, _ = exe(p_mm, s_mm, tokens, labels, cos, sin)
    # Adam's update is about lr * sign(gradient) in the first steps, so rounding differences
    # between the two runs (bf16, other summation order over microbatches) may move single
    # elements by up to 2 * lr per step; a wrong tile or a missing reduction moves them by far more
    lr, nsteps = 1e-3, 2
    ok, worst = True, 0.0
    for k, (got, want) in enumerate([(loss2, loss_ref2)] + list(zip(pytree.tree_leaves(p_mm2), pytree.tree_leaves(p_ref2)))):
        got.wait()
        for d, tile in got.local_tiles().items():
            lo, hi = tile_box(got.sharding, d - got.sharding["device_start"])
            ref = want[tuple(slice(a, b) for a, b in zip(lo, hi))] if want.dim() else want
            err = (tile.float() - ref.float()).abs().max().item()
            limit = 2e-2 * abs(float(ref)) if k == 0 else 2.5 * lr * nsteps + 8e-3 * ref.float().abs().max().item()
            worst = max(worst, err / limit)
            if err > limit:
                ok = False
    status = K.read_status()
    pm = getattr(exe, "_peer_moe", None)
    moe_calls = sum(o.calls for o in pm._ops.values()) if pm is not None else 0
    pc = getattr(exe, "_peer_comm", None)
    comm_calls = sum(o.calls for o in pc._ops.values()) if pc is not None else 0
    ft = getattr(exe, "_fused_tp", None)
    fused = {}
    for key, o in (ft._ops.items() if ft is not None else ()):
        kind = key[0] if isinstance(key[0], str) else "ar"
        fused[kind] = fused.get(kind, 0) + o.calls
    pr = getattr(exe, "_peer_reshard", None)
    peer_uses = sum(s["uses"] for s in pr.slots.values() if s) if pr is not None else 0
    flag = torch.tensor([1 if (ok and status == 0) else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    direct = torch.tensor([pr.direct_uses if pr is not None else 0, pr.copied_uses if pr is not None else 0], device=dev)
    dist.all_reduce(direct, op=dist.ReduceOp.SUM)
    uses = torch.tensor([peer_uses], device=dev)
    dist.all_reduce(uses, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"STEP_OK": bool(flag.item()), "worst_err_over_limit_rank0": worst, "peer_reshard_uses": int(uses.item()), "reshard_sources_written_in_place": int(direct[0].item()), "reshard_sources_copied": int(direct[1].item()), "peer_moe_calls": moe_calls, "peer_collective_calls": comm_calls, "fused_calls": fused,
                          "status": status, "native": exe.native_report() if hasattr(exe, "native_report") else {}, "loss": float(loss2.full_tensor().item()) if pp == 1 else None}), flush=True)
    dist.barrier()
    exe.shutdown()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
