"""Helpers for ``torch.nn`` models: modules as tasks, axis-annotated parameters and a
ready-made training step.

Counterpart of the Flax helpers of the reference (``multimesh/jax/flax/task.py:28-302``):

* :func:`task` wraps a module *class* so that every call of an instance runs as a task;
* :func:`shard_axes` attaches logical axis names to a parameter (the role of
  ``nn.with_partitioning``); :func:`parallelize_step` turns them into sharding constraints;
* :func:`parallelize_step` combines a model whose forward returns the loss with an optimizer
  rule into one compiled step ``(state, batch) -> (loss, state)``, compiles it ahead of time
  with compiler-chosen layouts and returns the step, the sharded initial state, the mesh and
  (for per-process batches) a ``prepare_batch`` function.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Sequence, Tuple, Type

import torch

from . import lib
from .task import MultiMesh, Task, TaskMesh, microbatch as _microbatch, register_task, task as _task, value_and_grad

_AXES_ATTR = "_mm_logical_axes"


def task(model: Type[torch.nn.Module], name: Optional[str] = None, *, task: Optional[Task] = None,
         mesh: Optional[TaskMesh] = None, devices: Optional[Sequence[int]] = None,
         logical_axes: Sequence[Tuple[str, str]] = (), split_backprop: Optional[Tuple[str, str]] = None):
    """Returns a subclass of ``model`` whose ``forward`` runs as the task ``name``.

    With ``task=`` (a :class:`Task` carrying a mesh or a mesh slice of the enclosing
    :class:`MultiMesh`) the placement is registered under the task's name when the module is
    called; otherwise ``mesh`` / ``devices`` place it explicitly."""
    base = name or (task.name if task is not None and task.name else model.__name__)

    class TaskModule(model):  # type: ignore[misc, valid-type]
        _mm_task_name = base

        def __call__(self, *args, **kwargs):
            call = super().__call__
            if task is not None:
                from .task import named_scope
                register_task(base, task=task)
                with named_scope(base):
                    return call(*args, **kwargs)
            fn = _task(lambda *a, **k: call(*a, **k), name=base, mesh=mesh, devices=devices,
                       logical_axes=logical_axes, split_backprop=split_backprop)
            return fn(*args, **kwargs)

    TaskModule.__name__ = model.__name__
    TaskModule.__qualname__ = model.__qualname__
    return TaskModule


def shard_axes(param: torch.Tensor, *names) -> torch.Tensor:
    """Attaches one logical axis name (or ``None``) per dimension to ``param``. The names are
    resolved per task through ``Task.logical_axes`` when the step is compiled."""
    if len(names) > param.dim():
        raise ValueError(f"{len(names)} axis names for a parameter with {param.dim()} dimensions")
    setattr(param, _AXES_ATTR, tuple(names) + (None,) * (param.dim() - len(names)))
    return param


def logical_axes_of(model: torch.nn.Module) -> Dict[str, Tuple]:
    return {n: getattr(p, _AXES_ATTR) for n, p in model.named_parameters() if hasattr(p, _AXES_ATTR)}


@dataclass
class SGD:
    lr: float = 1e-2

    def init(self, params):
        return {}

    def update(self, params, grads, opt_state, step):
        return {k: p - self.lr * grads[k] for k, p in params.items()}, opt_state


@dataclass
class AdamW:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0

    def init(self, params):
        return {"m": {k: torch.zeros_like(p) for k, p in params.items()},
                "v": {k: torch.zeros_like(p) for k, p in params.items()}}

    def update(self, params, grads, opt_state, step):
        t = step + 1
        new_p, new_m, new_v = {}, {}, {}
        c1 = 1.0 - self.beta1 ** t
        c2 = 1.0 - self.beta2 ** t
        for k, p in params.items():
            g = grads[k]
            m = self.beta1 * opt_state["m"][k] + (1 - self.beta1) * g
            v = self.beta2 * opt_state["v"][k] + (1 - self.beta2) * g * g
            upd = (m / c1) / (torch.sqrt(v / c2) + self.eps)
            new_p[k] = p - self.lr * (upd + self.weight_decay * p)
            new_m[k], new_v[k] = m, v
        return new_p, {"m": new_m, "v": new_v}


def parallelize_step(model: torch.nn.Module, optimizer: Any, mesh: Optional[MultiMesh] = None,
                     global_batch: Any = None, local_batch: Any = None, *, microbatch_size: Optional[int] = None,
                     schedule: str = "1f1b", backend: Optional[str] = None, num_devices: Optional[int] = None):
    """Builds and compiles ``step(state, batch) -> (loss, state)`` for ``model``, whose forward
    takes the batch (a tensor or a tuple) and returns the scalar loss.

    ``state`` is ``{"params", "opt", "step"}``. Exactly one of ``global_batch`` (an example of
    the full batch) or ``local_batch`` (an example of this process's share; the global batch is
    the concatenation over processes along dimension 0) must be given. Returns
    ``(compiled_step, init_state, mesh)`` or, for ``local_batch``,
    ``(compiled_step, init_state, mesh, prepare_batch)``."""
    from .compiler.api import compile_function
    if (global_batch is None) == (local_batch is None):
        raise ValueError("give exactly one of global_batch / local_batch")
    from torch.utils import _pytree as pytree
    nproc = 1
    if local_batch is not None:
        import torch.distributed as dist
        nproc = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        example = pytree.tree_map(lambda t: torch.empty((t.shape[0] * nproc,) + tuple(t.shape[1:]), dtype=t.dtype,
                                                        device="meta"), local_batch)
    else:
        example = pytree.tree_map(lambda t: torch.empty(t.shape, dtype=t.dtype, device="meta"), global_batch)
    axes = logical_axes_of(model)
    params0 = {n: p.detach() for n, p in model.named_parameters()}
    buffers = {n: b for n, b in model.named_buffers()}

    def loss_fn(params, batch):
        constrained = {n: (lib.with_sharding_constraint(p, axes[n]) if n in axes else p) for n, p in params.items()}
        args = batch if isinstance(batch, (tuple, list)) else (batch,)
        return torch.func.functional_call(model, {**constrained, **buffers}, tuple(args))

    def step(state, batch):
        vg = value_and_grad(loss_fn)
        if microbatch_size is not None:
            vg = _microbatch(vg, dim=0, size=microbatch_size, argnum=1, schedule=schedule)
        loss, grads = vg(state["params"], batch)
        new_params, new_opt = optimizer.update(state["params"], grads, state["opt"], state["step"])
        return loss, {"params": new_params, "opt": new_opt, "step": state["step"] + 1}

    state0 = {"params": params0, "opt": optimizer.init(params0), "step": torch.zeros((), dtype=torch.float32)}
    abstract_state = pytree.tree_map(lambda t: torch.empty(t.shape, dtype=t.dtype, device="meta"), state0)
    ctx = mesh if mesh is not None else lib.context()
    with lib.autoshard(True), ctx:
        compiled = compile_function(step, (abstract_state, example), mesh=mesh, donate_argnums=(0,), backend=backend,
                                    num_devices=num_devices, name=type(model).__name__ + "_step")
    init_state = compiled.shard_argument(0, state0)
    if global_batch is not None:
        return compiled, init_state, mesh

    def prepare_batch(local):
        """Assembles this process's share into the global batch layout of the compiled step."""
        if nproc == 1:
            return local
        import torch.distributed as dist

        def gather(t):
            parts = [torch.empty_like(t) for _ in range(nproc)]
            dist.all_gather(parts, t.contiguous())
            return torch.cat(parts, dim=0)
        return pytree.tree_map(gather, local)

    return compiled, init_state, mesh, prepare_batch
