"""Tutorial 3 - MultiMesh contexts for MPMD.

The model code stays unmodified: layers only carry named scopes. A ``MultiMesh`` is the global
device mesh *and* a registry of ``regex -> task`` rules; entering it applies the rules to every
scope name the capture sees (the backward pass of a scope becomes its own task ``<name>_bwd`` on
the same devices). ``mesh.slice(axis=i)`` gives the sub-mesh a task runs on; a factory can compute
the task from the matched text, which places a whole stack of layers with one rule.

Runs on four virtual CPU devices: ``python docs/tutorials/t03_multimesh_contexts.py``.
"""
import torch

import multimesh_jax_b200 as mm

LAYERS = 4


def loss_fn(weights, x, y):
    h = x
    for i, w in enumerate(weights):
        with mm.named_scope(f"layer.{i}"):
            h = torch.tanh(h @ w)
    with mm.named_scope("loss"):
        return ((h - y) ** 2).mean()


def step(weights, x, y):
    return mm.value_and_grad(loss_fn)(weights, x, y)


def main():
    mm.init(cpus=4)
    torch.manual_seed(0)
    weights = [torch.randn(8, 8) / 8 ** 0.5 for _ in range(LAYERS)]
    x, y = torch.randn(6, 8), torch.randn(6, 8)

    mesh = mm.MultiMesh((2, 2), ("stage", "model"))
    assert mesh.slice(stage=1).devices == [2, 3]

    def place(matched, backprop):
        # two layers per stage; the gradient task of a layer runs where its forward ran
        stage = int(matched.split(".")[1]) // 2
        return mm.Task(name=f"stage{stage}" + ("_bwd" if backprop else ""), mesh_slice={"stage": stage})

    with mesh:
        mesh.register_task(r"(layer\.\d+)", factory=place)
        mesh.register_task("(loss)", factory=lambda m, b: mm.Task(name="stage1" + ("_bwd" if b else ""),
                                                                   mesh_slice={"stage": 1}))
        exe = mm.compile_function(step, (weights, x, y), mesh=mesh, backend="cpu")
    loss, grads = exe(weights, x, y)
    with mm.ignore_transforms():
        ref_loss, ref_grads = step(weights, x, y)
    torch.testing.assert_close(loss.full_tensor(), ref_loss, rtol=1e-5, atol=1e-6)
    for g, r in zip(grads, ref_grads):
        torch.testing.assert_close(g.full_tensor(), r, rtol=1e-4, atol=1e-6)
    names = sorted({t["original_color"] for t in exe.plan["templates"]})
    print("tutorial 3: tasks", names)
    assert {"stage0", "stage1", "stage0_bwd", "stage1_bwd"} <= set(names)
    exe.shutdown()
    return names


if __name__ == "__main__":
    main()
