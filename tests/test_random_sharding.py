"""Randomised differential test of sharding propagation, SPMD lowering, reshard insertion and the
pipeline runtime: seeded random networks (MLP and attention blocks, norms, softmax, reductions over
the sequence, biases, concatenation, chunks, permutes, cumulative sums, flips, einsum, stack, expand) with random layout constraints on activations and weights, random logical ->
mesh axis tables (optionally a different priority order on odd stages), random three-axis meshes of
one to four stages, every pipeline schedule (zero-bubble with split backward tasks), interleaved
block placement, a first block that moves between stages per microbatch, recomputation on or off
and random microbatching, compiled for virtual CPU devices and compared with the eager step. The
method of the reference's Python end-to-end tests (tests/python/jax_task_test.py: same function with and
without the transformations), with the cases drawn instead of written. Longer runs of the same
generator found the microbatch-slice pairing error that ``test_sharding_e2e.py`` pins."""
import contextlib
import random

import pytest
import torch
from torch.utils import _pytree as pytree

import multimesh_jax_b200 as mm

OPS = ["mlp", "mlp", "tanh", "resid", "scale", "norm", "attn", "softmax", "meanseq", "gelu", "bias", "cat", "chunk",
       "permute", "cumsum", "max", "where", "clamp", "layernorm", "flip", "einsum", "stack", "expand", "sq_sum", "outer"]
MESHES = [(1, 2, 2), (2, 2, 1), (1, 4, 1), (2, 1, 2), (1, 2, 1), (2, 2, 2), (1, 1, 2), (4, 2, 1), (4, 1, 1), (3, 1, 2),
          (2, 1, 1)]
AXES = [("batch", "x"), ("hid", "y"), ("feat", "y"), ("seq", "y"), ("batch", "y"), ("hid", "x"), ("heads", "y"),
        ("heads", "x")]


def _draw(rng):
    mesh_shape = rng.choice(MESHES)
    B, S, D, F, H = rng.choice([4, 8]), rng.choice([2, 4]), rng.choice([8, 16]), rng.choice([8, 16]), rng.choice([2, 4])
    blocks = []
    for b in range(mesh_shape[0] * rng.randint(1, 3)):
        ops = [rng.choice(OPS) for _ in range(rng.randint(1, 4))]
        if b == 0 and not any(o in ("mlp", "scale", "attn", "bias") for o in ops):
            ops.append("mlp")
        constraints = [(rng.randint(0, len(ops)), (rng.choice([None, "batch"]), rng.choice([None, None, "seq"]),
                                                   rng.choice([None, None, "feat"]))) for _ in range(rng.randint(0, 2))]
        blocks.append((ops, constraints, rng.random() < 0.5))
    axes = list(AXES)
    rng.shuffle(axes)
    return dict(mesh_shape=mesh_shape, B=B, S=S, D=D, F=F, H=H, blocks=blocks, logical=axes[:rng.randint(1, 4)],
                microbatch=rng.choice([None, B // 2, B // 4 if B >= 8 else B // 2]),
                schedule=rng.choice(["gpipe", "1f1b", "zero-bubble-h2", "wavefront"]),
                other_order_on_odd_stages=rng.random() < 0.2, interleaved=rng.random() < 0.3,
                recompute=rng.choice([None, True, False]), moving_first_block=rng.random() < 0.15)


def _build(case):
    B, S, D, F, H = (case[k] for k in "BSDFH")
    g = torch.Generator().manual_seed(0)
    params = []
    for ops, _, _ in case["blocks"]:
        blk = []
        for op in ops:
            if op == "mlp":
                blk.append((torch.randn(D, F, generator=g) / D ** 0.5, torch.randn(F, D, generator=g) / F ** 0.5))
            elif op == "attn":
                blk.append((torch.randn(D, 3 * D, generator=g) / D ** 0.5, torch.randn(D, D, generator=g) / D ** 0.5))
            elif op in ("scale", "bias"):
                blk.append((torch.randn(D, generator=g),))
            else:
                blk.append(())
        params.append(blk)
    batch = (torch.randn(B, S, D, generator=g), torch.randn(B, S, D, generator=g))

    def loss_fn(params, batch):
        h, target = batch
        for bi, ((ops, constraints, shard_weights), blk) in enumerate(zip(case["blocks"], params)):
            with mm.named_scope(f"blk.{bi}"):
                for oi, (op, p) in enumerate(zip(ops, blk)):
                    for at, spec in constraints:
                        if at == oi:
                            h = mm.with_sharding_constraint(h, spec)
                    if op == "mlp":
                        w1, w2 = p
                        if shard_weights:
                            w1 = mm.with_sharding_constraint(w1, (None, "hid"))
                            w2 = mm.with_sharding_constraint(w2, ("hid", None))
                        h = h + torch.tanh(h @ w1) @ w2
                    elif op == "attn":
                        wqkv, wo = p
                        if shard_weights:
                            wqkv = mm.with_sharding_constraint(wqkv, (None, "heads"))
                            wo = mm.with_sharding_constraint(wo, ("heads", None))
                        b_, s_, _ = h.shape
                        qkv = (h @ wqkv).view(b_, s_, 3, H, D // H)
                        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
                        att = torch.softmax((q @ k.transpose(-1, -2)) / (D // H) ** 0.5, dim=-1)
                        h = h + (att @ v).transpose(1, 2).reshape(b_, s_, D) @ wo
                    elif op == "tanh":
                        h = torch.tanh(h)
                    elif op == "gelu":
                        h = torch.nn.functional.gelu(h)
                    elif op == "resid":
                        h = h + h * 0.5
                    elif op == "scale":
                        h = h * p[0]
                    elif op == "bias":
                        h = h + p[0]
                    elif op == "norm":
                        h = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + 1e-5)
                    elif op == "softmax":
                        h = torch.softmax(h, dim=-1) * h.shape[-1] ** 0.5
                    elif op == "meanseq":
                        h = h - h.mean(1, keepdim=True)
                    elif op == "cat":
                        h = torch.cat([h[..., h.shape[-1] // 2:] * 2.0, h[..., : h.shape[-1] // 2]], dim=-1)
                    elif op == "chunk":
                        lo, hi = h.chunk(2, dim=-1)
                        h = torch.cat([lo + hi, lo - hi], dim=-1)
                    elif op == "permute":
                        h = (h.permute(0, 2, 1).contiguous() * 1.5).permute(0, 2, 1)
                    elif op == "cumsum":
                        h = h + 0.1 * torch.cumsum(h, dim=1)
                    elif op == "max":
                        h = h - h.max(dim=-1, keepdim=True).values
                    elif op == "where":
                        h = torch.where(h > 0, h, 0.2 * h)
                    elif op == "clamp":
                        h = h.clamp(-1.5, 1.5)
                    elif op == "layernorm":
                        h = torch.nn.functional.layer_norm(h, (h.shape[-1],))
                    elif op == "flip":
                        h = h + 0.3 * h.flip(1)
                    elif op == "einsum":
                        h = h + 0.1 * torch.einsum("bsd,btd->bsd", h, h) / h.shape[1]
                    elif op == "stack":
                        h = torch.stack([h, 2.0 * h], dim=0).sum(0)
                    elif op == "expand":
                        h = h + h.mean(-1, keepdim=True).expand_as(h)
                    elif op == "sq_sum":
                        h = h / (1.0 + (h * h).sum((1, 2), keepdim=True)).sqrt()
                    elif op == "outer":
                        h = h + 0.05 * (h.unsqueeze(-1) * h.unsqueeze(-2)).sum(-1)
        with mm.named_scope("lossfn"):
            return ((h - target) ** 2).sum()

    def step(params, batch):
        vg = mm.value_and_grad(loss_fn)
        if case["microbatch"]:
            vg = mm.microbatch(vg, size=case["microbatch"], argnum=1, schedule=case["schedule"])
        return vg(params, batch)
    return step, params, batch


def _mesh(case):
    stages = case["mesh_shape"][0]
    blocks = len(case["blocks"])
    per_stage = blocks // stages
    split = ("_act", "_wgt") if case["schedule"] == "zero-bubble-h2" else None

    def axes_of(stage):
        if case["other_order_on_odd_stages"] and stage % 2:
            return list(reversed(case["logical"]))
        return case["logical"]

    def stage_of(block):       # interleaved: every microbatch visits each stage several times
        return block % stages if case["interleaved"] else block // per_stage

    def name_of(block, backprop):
        return (f"v{block}" if case["interleaved"] else f"s{stage_of(block)}") + ("_bwd" if backprop else "")

    def block_task(matched, backprop):
        block = int(matched.split(".")[1])
        if case["moving_first_block"] and block == 0 and not backprop and stages > 1 and not case["interleaved"]:
            # the first block's forward task runs on another stage's devices every microbatch
            return mm.Task(name="moving", mesh_slice={"stage": 0}, logical_axes=case["logical"],
                           loop_dependent_mesh_slice=lambda i: {"stage": i % stages})
        stage = stage_of(block)
        return mm.Task(name=name_of(block, backprop), mesh_slice={"stage": stage}, logical_axes=axes_of(stage),
                       split_backprop=split)

    last = stage_of(blocks - 1)
    mesh = mm.MultiMesh(case["mesh_shape"], ("stage", "x", "y"))
    mesh.register_task(r"(blk\.\d+)", factory=block_task)
    mesh.register_task("(lossfn)", factory=lambda m, b: mm.Task(name=name_of(blocks - 1, b), mesh_slice={"stage": last},
                                                                 logical_axes=axes_of(last), split_backprop=split))
    return mesh


@pytest.mark.parametrize("seed", range(32))
def test_random_network_and_layouts_match_the_eager_step(seed):
    mm.init(cpus=8)
    case = _draw(random.Random(1000 + seed))
    step, params, batch = _build(case)
    with mm.ignore_transforms():
        ref_loss, ref_grads = step(params, batch)
    mesh = _mesh(case)
    recompute = mm.enable_recomputation(case["recompute"]) if case["recompute"] is not None else contextlib.nullcontext()
    with mesh, recompute:
        exe = mm.compile_function(step, (params, batch), mesh=mesh, backend="cpu")
    try:
        loss, grads = exe(params, batch)
        scale = float(ref_loss.abs())
        assert abs(float(loss.full_tensor()) - float(ref_loss)) <= 1e-4 * scale + 1e-5, case
        for got, want in zip(pytree.tree_leaves(grads), pytree.tree_leaves(ref_grads)):
            err = float((got.full_tensor() - want).abs().max())
            assert err <= 2e-3 * (float(want.abs().max()) + 1e-3 * scale), (err, case)
    finally:
        exe.shutdown()
