"""Tutorial 2 - logical autosharding for MPMD.

Two calls of the same layer are assigned to two different sub-meshes. Each task carries its own
mapping from logical axes to mesh axes, so the first stage can be tensor parallel while the second
is data parallel; the activation that crosses the boundary is re-laid-out automatically (a reshard
from the first sub-mesh's layout to the second's).

Runs on four virtual CPU devices: ``python docs/tutorials/t02_mpmd_autosharding.py``.
"""
import torch

import multimesh_jax_b200 as mm


def layer(w, x):
    w = mm.with_sharding_constraint(w, ("hidden", None))
    x = mm.with_sharding_constraint(x, ("batch", None))
    return torch.tanh(x @ w.t())


def model(w1, w2, x):
    with mm.named_scope("first"):
        h = layer(w1, x)
    with mm.named_scope("second"):
        return layer(w2, h).sum()


def main():
    mm.init(cpus=4)
    torch.manual_seed(0)
    w1, w2, x = torch.randn(16, 8), torch.randn(8, 16), torch.randn(12, 8)

    mesh = mm.MultiMesh((2, 2), ("stage", "x"))
    with mesh:
        # stage 0 shards the features (tensor parallel), stage 1 shards the batch (data parallel)
        mesh.register_task("first", task=mm.Task(mesh_slice={"stage": 0}, logical_axes=[("hidden", "x")]))
        mesh.register_task("second", task=mm.Task(mesh_slice={"stage": 1}, logical_axes=[("batch", "x")]))
        exe = mm.compile_function(model, (w1, w2, x), mesh=mesh, backend="cpu")
    out = exe(w1, w2, x)
    with mm.ignore_transforms():
        ref = model(w1, w2, x)
    torch.testing.assert_close(out.full_tensor(), ref, rtol=1e-5, atol=1e-5)

    tasks = [(op["name"], op["device_start"], op["num_devices"]) for op in exe.plan["ops"] if op["kind"] == "task"]
    reshards = sum(1 for op in exe.plan["ops"] if op["kind"] == "reshard")
    assert [t[1:] for t in tasks] == [(0, 2), (2, 2)] and reshards >= 1
    print("tutorial 2: tasks", tasks, "reshards", reshards)
    exe.shutdown()
    return tasks


if __name__ == "__main__":
    main()
