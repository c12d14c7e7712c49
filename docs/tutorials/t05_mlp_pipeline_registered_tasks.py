"""Tutorial 5 - an MLP pipeline with external task registration.

The model is an ordinary ``torch.nn.Module`` with no task transforms in it. Scope names come from
the module tree (``mm.module_scopes``), and the placement is registered from the outside with
regular expressions, so the same model code can be run single-device, as a 2-stage or as a 4-stage
pipeline by changing only the registration. The step uses the zero-bubble schedule: the backward
task of every stage is split into the half that produces the gradient for the previous stage and
the half that produces weight gradients, which the scheduler uses to fill the pipeline bubbles.

Runs on four virtual CPU devices: ``python docs/tutorials/t05_mlp_pipeline_registered_tasks.py``.
"""
import torch

import multimesh_jax_b200 as mm

DEPTH, D = 8, 16


class MLP(torch.nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.layers = torch.nn.ModuleList(torch.nn.Linear(D, D, bias=False) for _ in range(DEPTH))

    def forward(self, x):
        for layer in self.layers:
            x = torch.tanh(layer(x))
        return x


def make_step(net, names, microbatch, schedule):
    def loss_fn(params, batch):
        x, y = batch
        with mm.module_scopes(net):          # scope names "layers.0", "layers.1", ... from the module tree
            out = torch.func.functional_call(net, dict(zip(names, params)), (x,))
        with mm.named_scope("loss"):
            return ((out - y) ** 2).sum()

    def step(params, batch):
        vg = mm.microbatch(mm.value_and_grad(loss_fn), size=microbatch, argnum=1, schedule=schedule)
        loss, grads = vg(params, batch)
        return loss, [p - 0.05 * g for p, g in zip(params, grads)]
    return step


def main(stages=4):
    mm.init(cpus=stages)
    net = MLP()
    names = [n for n, _ in net.named_parameters()]
    params = [p.detach().clone() for _, p in net.named_parameters()]
    torch.manual_seed(1)
    batch = (torch.randn(16, D), torch.randn(16, D))
    step = make_step(net, names, microbatch=2, schedule="zero-bubble-h2")

    per_stage = DEPTH // stages
    split = ("_act", "_wgt")                 # suffixes of the two halves of every backward task

    def place(matched, backprop):
        s = int(matched.split(".")[1]) // per_stage
        return mm.Task(name=f"stage{s}" + ("_bwd" if backprop else ""), mesh_slice={"stage": s}, split_backprop=split)

    mesh = mm.MultiMesh((stages,), ("stage",))
    with mesh:
        mesh.register_task(r"(layers\.\d+)", factory=place)
        mesh.register_task("(loss)", factory=lambda m, b: mm.Task(name=f"stage{stages - 1}" + ("_bwd" if b else ""),
                                                                   mesh_slice={"stage": stages - 1},
                                                                   split_backprop=split))
        exe = mm.compile_function(step, (params, batch), mesh=mesh, backend="cpu")
    loss, new_params = exe(params, batch)
    with mm.ignore_transforms():
        ref_loss, ref_params = step(params, batch)
    torch.testing.assert_close(loss.full_tensor(), ref_loss, rtol=1e-4, atol=1e-5)
    for a, b in zip(new_params, ref_params):
        torch.testing.assert_close(a.full_tensor(), b, rtol=1e-4, atol=1e-5)
    loop = [t for t in exe.plan["templates"] if t["in_loop"]]
    deferred = sorted(t["name"].split(".", 1)[1] for t in loop if t["noncritical"])
    print("tutorial 5:", len(loop), "loop tasks; weight-gradient halves", deferred, "schedule", exe.plan["stats"]["schedule"])
    assert len(deferred) == stages - 1
    exe.shutdown()
    return deferred


if __name__ == "__main__":
    main()
