"""Randomised differential test of task placement: seeded random DAGs of explicit tasks
(``mm.task``) on arbitrary, possibly overlapping sub-meshes of six virtual devices - one or two
mesh axes, random logical-axis tables, layout constraints on activations and weights - with
uncoloured operators between the tasks, values read by several later tasks and one or two results,
with and without the backward pass and the recomputation pass. Colouring, grouping, recolouring,
reshard insertion between unequal meshes, sharding propagation and execution are checked against
the eager function (the reference compares the same function with and without its transformations:
tests/python/jax_task_test.py, tests/python/jax_auto_task_test.py)."""
import contextlib
import random

import pytest
import torch
from torch.utils import _pytree as pytree

import multimesh_jax_b200 as mm

DEVICES = 6


def _draw(rng):
    tasks = []
    for _ in range(rng.randint(2, 5)):
        n = rng.choice([1, 1, 2, 2, 3, 4])
        dims = rng.choice([(n,), (n,)] + ([(2, n // 2)] if n == 4 else []))
        tasks.append(dict(n=n, start=rng.randint(0, DEVICES - n), dims=dims, axes=("x", "y")[:len(dims)],
                          logical=rng.sample([("batch", "x"), ("feat", "x"), ("hid", "x"), ("hid", "y"), ("batch", "y")],
                                             rng.randint(0, 2)),
                          body=[rng.choice(["mlp", "tanh", "scale", "norm", "resid", "softmax"]) for _ in range(rng.randint(1, 3))],
                          operands=[rng.randrange(10 ** 6) for _ in range(rng.randint(1, 2))],
                          constraint=rng.choice([None, ("batch", None), (None, "feat"), ("batch", "feat")]),
                          shard_weights=rng.random() < 0.5))
    return dict(tasks=tasks, between=[rng.choice([None, "tanh", "add_input", "double", "neg"]) for _ in tasks],
                results=rng.randint(1, 2), B=rng.choice([4, 8, 12]), D=rng.choice([8, 12]), F=rng.choice([8, 16]),
                backward=rng.random() < 0.7, recompute=rng.choice([None, True, False]))


def _build(case, seed):
    B, D, F = case["B"], case["D"], case["F"]
    g = torch.Generator().manual_seed(seed)
    params = []
    for t in case["tasks"]:
        params.append([(torch.randn(D, F, generator=g) / D ** 0.5, torch.randn(F, D, generator=g) / F ** 0.5) if op == "mlp"
                       else (torch.randn(D, generator=g),) if op == "scale" else () for op in t["body"]])
    x = torch.randn(B, D, generator=g)

    def body_of(index, t):
        def body(p, *operands):
            h = operands[0]
            for extra in operands[1:]:
                h = h + 0.5 * extra
            if t["constraint"] is not None:
                h = mm.with_sharding_constraint(h, t["constraint"])
            for op, weights in zip(t["body"], p):
                if op == "mlp":
                    w1, w2 = weights
                    if t["shard_weights"]:
                        w1 = mm.with_sharding_constraint(w1, (None, "hid"))
                        w2 = mm.with_sharding_constraint(w2, ("hid", None))
                    h = h + torch.tanh(h @ w1) @ w2
                elif op == "tanh":
                    h = torch.tanh(h)
                elif op == "scale":
                    h = h * weights[0]
                elif op == "norm":
                    h = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + 1e-5)
                elif op == "resid":
                    h = h + 0.5 * h
                elif op == "softmax":
                    h = torch.softmax(h, -1) * 3.0
            return h
        mesh = mm.TaskMesh(t["dims"], t["axes"], list(range(t["start"], t["start"] + t["n"])))
        return mm.task(body, name=f"t{index}", mesh=mesh, logical_axes=t["logical"])

    bodies = [body_of(i, t) for i, t in enumerate(case["tasks"])]

    def forward(params, x):
        values = [x]
        for i, (t, body) in enumerate(zip(case["tasks"], bodies)):
            out = body(params[i], *[values[k % len(values)] for k in t["operands"]])
            glue = case["between"][i]               # operators that belong to no task
            if glue == "tanh":
                out = torch.tanh(out)
            elif glue == "add_input":
                out = out + values[0]
            elif glue == "double":
                out = out * 2.0
            elif glue == "neg":
                out = -out
            values.append(out)
        return sum((o ** 2).sum() for o in values[-case["results"]:])

    step = (lambda params, x: mm.value_and_grad(forward)(params, x)) if case["backward"] else forward
    return step, params, x


def _cases(count):
    """The first `count` seeds whose result depends on at least one parameter (a drawn graph may
    return values that no parametrised task feeds; its backward pass would have nothing to do)."""
    seeds, seed = [], 0
    while len(seeds) < count:
        case = _draw(random.Random(5000 + seed))
        forward, params, x = _build(dict(case, backward=False), seed)
        for p in pytree.tree_leaves(params):
            p.requires_grad_(True)
        with mm.ignore_transforms():
            if not case["backward"] or forward(params, x).requires_grad:
                seeds.append(seed)
        seed += 1
    return seeds


@pytest.mark.parametrize("seed", _cases(16))
def test_random_task_graph_matches_the_eager_function(seed):
    mm.init(cpus=DEVICES)
    case = _draw(random.Random(5000 + seed))
    step, params, x = _build(case, seed)
    with mm.ignore_transforms():
        want = step(params, x)
    recompute = mm.enable_recomputation(case["recompute"]) if case["recompute"] is not None else contextlib.nullcontext()
    with recompute:
        exe = mm.compile_function(step, (params, x), num_devices=DEVICES, backend="cpu")
    try:
        got = exe(params, x)
        want_leaves, got_leaves = pytree.tree_leaves(want), pytree.tree_leaves(got)
        assert len(want_leaves) == len(got_leaves)
        scale = float(want_leaves[0].abs()) + 1e-6
        for a, b in zip(got_leaves, want_leaves):
            a = a.full_tensor() if hasattr(a, "full_tensor") else a
            err = float((a - b).abs().max())
            assert err <= 2e-3 * (float(b.abs().max()) + 1e-3 * scale), (err, case)
    finally:
        exe.shutdown()
