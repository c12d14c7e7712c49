"""Tutorial 4 - an MLP pipeline with task transforms on modules.

``mm.nn.task(ModuleClass, name, devices=...)`` wraps a module class so that every call of an
instance runs as a task on the given devices; the backward pass of each instance becomes the task
``<name>_bwd`` on the same devices. ``shard_axes`` names the dimensions of a parameter, and
``parallelize_step`` builds the whole training step - value and gradient over microbatches, the
optimizer update, ahead-of-time compilation - and returns it with the initial (sharded) state.

Runs on two virtual CPU devices: ``python docs/tutorials/t04_mlp_pipeline_module_tasks.py``.
"""
import torch

import multimesh_jax_b200 as mm
from multimesh_jax_b200 import nn as mmnn


class Block(torch.nn.Module):
    """Dense layer + tanh; the output features carry the logical axis "hidden"."""

    def __init__(self, d_in, d_out):
        super().__init__()
        self.w = torch.nn.Parameter(torch.randn(d_out, d_in) / d_in ** 0.5)
        mmnn.shard_axes(self.w, "hidden", None)

    def forward(self, x):
        return torch.tanh(torch.nn.functional.linear(x, self.w))


class Pipeline(torch.nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.first = mmnn.task(Block, "first", devices=[0])(8, 32)     # stage 0 on device 0
        self.second = mmnn.task(Block, "second", devices=[1])(32, 4)   # stage 1 on device 1

    def forward(self, x, y):
        return ((self.second(self.first(x)) - y) ** 2).mean()


def main(steps=5):
    mm.init(cpus=2)
    torch.manual_seed(1)
    x, y = torch.randn(16, 8), torch.randn(16, 4)
    net = Pipeline()
    # four microbatches of four rows, forward and backward tasks interleaved one-forward-one-backward
    compiled, state, mesh = mmnn.parallelize_step(net, mmnn.SGD(lr=0.2), None, global_batch=(x, y), microbatch_size=4,
                                                  schedule="1f1b", backend="cpu", num_devices=2)
    losses = []
    for _ in range(steps):
        loss, state = compiled(state, (x, y))
        losses.append(float(loss.full_tensor()))
    tasks = sorted({t["original_color"] for t in compiled.plan["templates"] if t["in_loop"]})
    print("tutorial 4: loop tasks", tasks, "losses", [round(v, 4) for v in losses])
    assert tasks == ["first", "first_bwd", "second", "second_bwd"] and losses[-1] < losses[0]
    compiled.shutdown()
    return losses


if __name__ == "__main__":
    main()
