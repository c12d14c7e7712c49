"""Tutorial 1 - logical autosharding for SPMD.

Model code names tensor dimensions with *logical* axes ("batch", "hidden", ...). A task maps the
logical names to the axes of its device mesh, in priority order; the compiler derives the physical
layout of every tensor in the task from those few annotations and inserts the collectives the
layouts imply. The model code itself never mentions devices.

Runs on four virtual CPU devices: ``python docs/tutorials/t01_spmd_autosharding.py``.
"""
import torch

import multimesh_jax_b200 as mm


def layer(w, x):
    # "hidden" names the output features of the projection, "batch" the rows of the activations
    w = mm.with_sharding_constraint(w, ("hidden", None))
    x = mm.with_sharding_constraint(x, ("batch", None))
    return torch.relu(x @ w.t())


def model(w1, w2, x):
    with mm.named_scope("mlp"):
        return layer(w2, layer(w1, x)).sum()


def main():
    mm.init(cpus=4)
    torch.manual_seed(0)
    w1, w2, x = torch.randn(16, 8), torch.randn(8, 16), torch.randn(12, 8)

    # one task on the whole 2 x 2 mesh: rows of the batch over "data", features over "model"
    mesh = mm.MultiMesh((2, 2), ("data", "model"))
    task = mm.Task(mesh_slice={}, logical_axes=[("batch", "data"), ("hidden", "model")])   # empty slice = whole mesh
    with mesh:
        mesh.register_task("mlp", task=task)
        exe = mm.compile_function(model, (w1, w2, x), mesh=mesh, backend="cpu")
    out = exe(w1, w2, x)

    # the same function with every transform switched off is the single-device reference
    with mm.ignore_transforms():
        ref = model(w1, w2, x)
    torch.testing.assert_close(out.full_tensor(), ref, rtol=1e-5, atol=1e-5)

    # what the compiler chose for the arguments: w1 [16, 8] is split 2-way along its first dimension
    layouts = [s for s in exe.input_shardings() if s is not None]
    w1_layout = next(s for s in layouts if s["sizes"] == [16, 8])
    assert w1_layout["shard_size"] == [8, 8]
    print("tutorial 1: result", float(out.full_tensor()), "w1 tile", w1_layout["shard_size"])
    exe.shutdown()
    return float(out.full_tensor())


if __name__ == "__main__":
    main()
