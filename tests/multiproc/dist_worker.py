"""Worker of the multi-process tests (gloo ranks on CPU, one process per virtual device).

Modes:
  step   - pipeline x data x tensor parallel training step through the "dist" topology; every rank
           checks its tiles of the loss and of the updated parameters against the eager step.
  leave  - the last rank exits cleanly between steps; the others see their next collective
           end with an error within the process-group timeout and report it as a status.
  moving - a forward task that runs on another stage's devices every microbatch (one template on two
           device ranges) with a layout change inside; every rank checks its tiles against eager.
  ckpt   - every rank saves its tiles of the updated parameters, the job reloads them (stored layout
           and the compiled step's layout) and compares; the manifest names only complete tiles.
"""
import datetime
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def build(pp, tp, dp=1):
    import multimesh_jax_b200 as mm
    from multimesh_jax_b200.models import llama
    torch.manual_seed(0)
    cfg = llama.LlamaConfig.tiny(n_layers=2 * pp, n_heads=4, n_kv_heads=2, d_model=64, d_ff=96, vocab=128)
    cfg.dtype = torch.float32
    B, S, MB = 8, 16, 4
    params = llama.init_params(cfg)
    state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    labels = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=MB)
    mesh = mm.MultiMesh((pp, dp, tp), ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=pp)
    args = (params, state, tokens, labels, cos, sin)
    with mesh:
        exe = mm.compile_function(step, args, mesh=mesh, backend="dist")
    return mm, exe, step, args


def mode_step(pp, tp, dp=1):
    from torch.utils import _pytree as pytree
    rank = dist.get_rank()
    mm, exe, step, args = build(pp, tp, dp)
    with mm.ignore_transforms():
        loss_ref, p_ref, _ = step(*args)
    loss, p_mm, _ = exe(*args)
    checked = 0
    for got, want in [(loss, loss_ref)] + list(zip(pytree.tree_leaves(p_mm), pytree.tree_leaves(p_ref))):
        got.wait()
        for d, tile in got.local_tiles().items():
            from multimesh_jax_b200.runtime.collectives import tile_box
            lo, hi = tile_box(got.sharding, d - got.sharding["device_start"])
            ref = want[tuple(slice(a, b) for a, b in zip(lo, hi))] if want.dim() else want
            torch.testing.assert_close(tile, ref, rtol=1e-3, atol=2e-4)
            checked += 1
    ok = torch.tensor([1 if checked > 0 else 0])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"DIST_STEP_OK": bool(ok.item()), "tiles_checked_rank0": checked}), flush=True)
    exe.shutdown()


def mode_moving():
    import multimesh_jax_b200 as mm
    from multimesh_jax_b200.runtime.collectives import tile_box
    rank = dist.get_rank()
    g = torch.Generator().manual_seed(0)
    B, S, D, F = 8, 4, 16, 8
    params = [torch.randn(D, F, generator=g) / 4, torch.randn(F, D, generator=g) / 3, torch.randn(D, generator=g)]
    batch = (torch.randn(B, S, D, generator=g), torch.randn(B, S, D, generator=g))

    def loss_fn(params, batch):
        (w1, w2, scale), (x, y) = params, batch
        with mm.named_scope("blk.0"):
            h = mm.with_sharding_constraint(x, (None, "seq", None))
            h = h + torch.tanh(h @ w1) @ w2
        with mm.named_scope("blk.1"):
            h = h * scale
            return ((h - y) ** 2).sum()

    def step(params, batch):
        return mm.microbatch(mm.value_and_grad(loss_fn), size=2, argnum=1, schedule="1f1b")(params, batch)

    axes = [("seq", "model")]

    def factory(matched, backprop):
        i = int(matched.split(".")[1])
        if i == 0 and not backprop:
            return mm.Task(name="moving", mesh_slice={"stage": 0}, logical_axes=axes,
                           loop_dependent_mesh_slice=lambda k: {"stage": k % 2})
        return mm.Task(name=f"s{i}" + ("_bwd" if backprop else ""), mesh_slice={"stage": i}, logical_axes=axes)

    mesh = mm.MultiMesh((2, 2), ("stage", "model"))
    mesh.register_task(r"(blk\.\d+)", factory=factory)
    with mesh:
        exe = mm.compile_function(step, (params, batch), mesh=mesh, backend="dist")
    with mm.ignore_transforms():
        ref_loss, ref_grads = step(params, batch)
    loss, grads = exe(params, batch)
    checked = 0
    for got, want in [(loss, ref_loss)] + list(zip(grads, ref_grads)):
        got.wait()
        for d, tile in got.local_tiles().items():
            lo, hi = tile_box(got.sharding, d - got.sharding["device_start"])
            ref = want[tuple(slice(a, b) for a, b in zip(lo, hi))] if want.dim() else want
            torch.testing.assert_close(tile, ref, rtol=1e-4, atol=1e-4)
            checked += 1
    moved_here = sum(1 for op in exe.plan["ops"] if op["kind"] == "task" and op["name"].endswith("moving_loop")
                     and op["device_start"] <= rank < op["device_start"] + op["num_devices"])
    ok = torch.tensor([1 if moved_here == 2 else 0])      # four microbatches: two on each stage's devices
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"DIST_MOVING_OK": bool(ok.item()), "tiles_checked_rank0": checked}), flush=True)
    exe.shutdown()


def mode_ckpt(pp, tp, directory):
    from torch.utils import _pytree as pytree
    from multimesh_jax_b200.utils import checkpoint
    from multimesh_jax_b200.runtime.executable import ShardedTensor
    rank = dist.get_rank()
    mm, exe, step, args = build(pp, tp)
    loss, p_mm, s_mm = exe(*args)
    loss.wait()
    manifest = checkpoint.save(directory, {"params": p_mm, "step": 3}, step=3)
    # after save() returns on any rank the manifest exists and every file it names is complete
    assert os.path.exists(os.path.join(directory, checkpoint.MANIFEST))
    names = {t["file"] for e in manifest["leaves"] if e["kind"] == "sharded" for t in e["tiles"]}
    assert all(os.path.exists(os.path.join(directory, n)) for n in names)
    assert not [f for f in os.listdir(directory) if ".tmp" in f]
    is_leaf = lambda x: isinstance(x, ShardedTensor)
    back = checkpoint.load(directory, topology=exe.topology)
    checked = 0
    for got, want in zip(pytree.tree_flatten(back["params"], is_leaf=is_leaf)[0],
                         pytree.tree_flatten(p_mm, is_leaf=is_leaf)[0]):
        assert "shard_size" in got.sharding and list(got.sharding["shard_size"]) == list(want.sharding["shard_size"])
        for d, tile in want.local_tiles().items():
            torch.testing.assert_close(got.tile(d), tile, rtol=0, atol=0)
            checked += 1
    ok = torch.tensor([1 if checked > 0 and back["step"] == 3 else 0])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"DIST_CKPT_OK": bool(ok.item()), "tiles_checked_rank0": checked}), flush=True)
    exe.shutdown()


def mode_leave(pp, tp):
    rank, world = dist.get_rank(), dist.get_world_size()
    mm, exe, step, args = build(pp, tp)
    loss, params, state = exe(*args)
    loss.wait()
    dist.barrier()
    if rank == world - 1:
        # leaves between steps, with nothing in flight
        exe.shutdown()
        print(json.dumps({"rank": rank, "left": True}), flush=True)
        os._exit(0)
    t0 = time.time()
    try:
        loss, params, state = exe(*args)
        for leaf in [loss]:
            leaf.wait()
        # ranks that never talk to the lost rank may finish the step; they learn at the barrier
        dist.barrier()
        outcome = "no error"
    except (mm.StepFailed, RuntimeError) as e:
        outcome = "error: " + type(e).__name__
    print(json.dumps({"rank": rank, "outcome": outcome, "seconds": round(time.time() - t0, 1)}), flush=True)
    os._exit(0)


if __name__ == "__main__":
    mode, pp, tp = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    dp = int(sys.argv[4]) if len(sys.argv) > 4 and mode == "step" else 1
    timeout = datetime.timedelta(seconds=8 if mode == "leave" else 120)
    dist.init_process_group("gloo", timeout=timeout)
    if mode == "step":
        mode_step(pp, tp, dp)
    elif mode == "ckpt":
        mode_ckpt(pp, tp, sys.argv[4])
    elif mode == "moving":
        mode_moving()
    else:
        mode_leave(pp, tp)
    dist.destroy_process_group()
