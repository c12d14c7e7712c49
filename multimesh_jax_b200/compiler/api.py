"""Compile entry points: ``compile_function`` (ahead of time) and ``JitFunction``.

Compilation = capture with torch.fx -> native graph -> native MPMD pipeline ->
plan -> per-task programs -> :class:`Executable`. Small single-task programs
take the *fast path* and run the captured graph directly, bypassing the MPMD
runtime, as the reference does for programs under 20 instructions
(``src/pjrt_client/mm_pjrt_client.cc:51, 587-617``).
"""
from __future__ import annotations

import os
from typing import Any, Callable, Dict, Optional, Sequence

import torch
from torch.utils import _pytree as pytree

from .. import state
from ..runtime.collectives import Topology
from ..runtime.executable import Executable, ShardedTensor
from ..runtime.wrapper import WrapperExecutable
from ..task import MultiMesh
from .capture import Captured, capture, make_partition

FAST_PATH_MAX_NODES = 20


def _partition_config(**overrides):
    from .. import _mm_C
    cfg = _mm_C.PartitionConfig.from_env()
    cfg.replicated_parameter_num_elements_cutoff = state.knobs["replicated_parameter_num_elements_cutoff"]
    cfg.recompute_from_arguments_if_cost_less_than = state.knobs["recompute_from_arguments_if_cost_less_than"]
    cfg.enable_recomputation = bool(state.flags.recomputation)
    if state.startup.dump:
        os.makedirs(state.startup.dump, exist_ok=True)
        cfg.dump_dir = state.startup.dump
        cfg.dump_all_passes = bool(state.startup.dump_all_passes)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


def _is_spec(x) -> bool:
    """One layout: a tuple / list with one entry per dimension, each None, an axis name or a tuple
    of axis names."""
    return isinstance(x, (tuple, list)) and all(
        e is None or isinstance(e, str) or (isinstance(e, (tuple, list)) and e and all(isinstance(a, str) for a in e))
        for e in x)


def _apply_shardings(cap: Captured, in_shardings, example_args) -> None:
    """Attaches user-given axis names to graph inputs (mesh-axis names unless autoshard).
    ``in_shardings`` has one entry per positional argument: ``None`` (the compiler's choice), one
    layout - applied to every tensor of that argument - or a container shaped like the argument
    that holds a layout or ``None`` per tensor."""
    if in_shardings is None:
        return
    example_args = tuple(example_args)
    if not isinstance(in_shardings, (tuple, list)) or len(in_shardings) != len(example_args):
        raise ValueError(f"in_shardings needs one entry per positional argument ({len(example_args)}), got {in_shardings!r}")
    from ..lib import _canonical_axes
    k = 0           # index over the tensor leaves of all arguments = index over graph inputs
    for pos, (arg, entry) in enumerate(zip(example_args, in_shardings)):
        leaves = [a for a in pytree.tree_leaves(arg) if isinstance(a, torch.Tensor)]
        if entry is None:
            specs = [None] * len(leaves)
        elif _is_spec(entry) and not (isinstance(arg, (tuple, list)) and len(entry) == len(arg) and
                                       all(e is None or _is_spec(e) for e in entry) and
                                       any(_is_spec(e) for e in entry)):
            specs = [entry] * len(leaves)
        else:
            specs = pytree.tree_leaves(entry, is_leaf=lambda x: x is None or _is_spec(x))
            if len(specs) != len(leaves):
                raise ValueError(f"in_shardings[{pos}] holds {len(specs)} layouts for {len(leaves)} tensors")
        for spec in specs:
            if spec is not None:
                vid = cap.graph.inputs[k]
                ndim = len(cap.graph.value(vid)["shape"])
                cap.graph.set_value_axes(vid, _canonical_axes(spec, ndim), bool(state.flags.autoshard))
            k += 1


def compile_function(fn: Callable, example_args: Sequence[Any], *, mesh: Optional[MultiMesh] = None,
                     num_devices: Optional[int] = None, donate_argnums: Sequence[int] = (),
                     backend: Optional[str] = None, in_shardings=None, context=None, topology: Optional[Topology] = None,
                     name: Optional[str] = None, config_overrides: Optional[Dict[str, Any]] = None,
                     save_program: Optional[str] = None):
    """Captures ``fn``, partitions it and returns the executable. ``save_program``: also write
    the captured step, before partitioning, to this path as a stored program that
    :func:`compile_program_file` can compile again without the model, its tensors or a device."""
    from .. import _mm_C
    mesh = mesh or MultiMesh.current()
    if num_devices is None:
        if mesh is not None:
            num_devices = mesh.size
        else:
            num_devices = max(1, state.startup.gpus or state.startup.cpus or 1)
    if topology is None:
        topology = Topology.auto(num_devices, backend)
    device = topology.torch_device(topology.local_devices[0])
    cap = capture(fn, example_args, device=device, mesh=mesh)
    _apply_shardings(cap, in_shardings, example_args)
    if donate_argnums:
        flat_idx = pytree.tree_unflatten(list(range(len(cap.input_is_tensor))), cap.in_spec)
        donated = []
        tensor_rank = {}
        k = 0
        for i, ok in enumerate(cap.input_is_tensor):
            if ok:
                tensor_rank[i] = k
                k += 1
        for a in donate_argnums:
            for pos in pytree.tree_leaves(flat_idx[a]):
                if pos in tensor_rank:
                    donated.append(tensor_rank[pos])
        cap.graph.set_donated_inputs(donated)
        cap.donated_inputs = donated
    nmb = cap.loop_configs[0]["num_microbatches"] if cap.loop_configs else 0
    part = make_partition(num_devices, mesh, nmb)
    cfg = _partition_config(**(config_overrides or {}))
    if save_program is not None:
        # before partitioning: the pipeline rewrites the graph in place
        _mm_C.save_program(cap.graph, part, cfg, str(save_program))
    plan = _mm_C.mpmd_partition(cap.graph, part, cfg)
    name = name or getattr(fn, "__name__", "step")
    reason = bypass_reason(cap, plan, num_devices, donate_argnums, context)
    if reason is not None:
        exe = WrapperExecutable(cap, plan, topology, name=name, reason=reason, num_devices=num_devices)
    else:
        exe = Executable(cap, plan, topology, context=context, name=name)
    exe.partition = part
    return exe


def compile_program_file(path: str, device_memory_bytes: int = 0, want_plan: bool = False) -> Dict[str, Any]:
    """Offline compile of a stored program (``compile_function(..., save_program=path)``): the
    whole MPMD pipeline in C++ plus a replay of the plan on the mock runtime. Returns the number
    of templates / tasks / reshards, the plan and operation hashes, per-device memory
    high-water marks, ``fits`` (high-water mark within ``device_memory_bytes``; 0 = no limit),
    the hazard report of the submission log and, with ``want_plan``, the plan itself.
    Counterpart of ``CompileHloModuleFromFile`` (src/pjrt_client/mm_pjrt_client.cc:702-771)."""
    from .. import _mm_C
    return _mm_C.compile_program_file(str(path), int(device_memory_bytes), bool(want_plan))


def bypass_reason(cap: Captured, plan: dict, num_devices: int, donate_argnums, context) -> Optional[str]:
    """Why a compiled program does not need the MPMD runtime, or None when it does.

    ``"fast-path"``: the plan is a single task without reshards, the program has fewer than
    ``FAST_PATH_MAX_NODES`` operators and none of them is a marker (``mm.*``: task, microbatch
    or sharding annotations) - ``src/pjrt_client/mm_pjrt_client.cc:587-617``.
    ``"single-device"``: the device assignment is one device and the program has no marker and
    no microbatch loop, so there is nothing to partition, schedule or reshard -
    ``src/pjrt_client/mm_pjrt_client.cc:525-534``.
    Both are switched off by ``enable_fast_path(False)`` (the differential test harness does
    that to force every program through the partitioner), by donated arguments (in-place
    reuse of their tiles is a service of the partitioned executable) and by an explicitly
    given runtime context (mock runs want to see the submissions)."""
    if not state.flags.fast_path or context is not None or donate_argnums or cap.loop_configs:
        return None
    g = cap.graph
    ops = [op for op in plan["ops"] if op["kind"] in ("task", "reshard")]
    if len(ops) != 1 or ops[0]["kind"] != "task":
        return None
    if any(t["name"].split(".", 1)[-1] != "global" for t in plan["templates"]):
        return None                      # the user placed the work in a task of their own
    node_ids = [n for t in plan["templates"] for n in t["nodes"]]
    names = [g.node(n)["op"] for n in node_ids]
    if any(nm.startswith("mm.") for nm in names):
        return None
    if any(len(ax) > 0 for sid in plan["param_stores"] + plan["root_stores"] if sid >= 0
           for ax in plan["stores"][sid]["shape"]["dim_axes"]):
        return None                      # a sharded argument or result: the partitioned path owns layouts
    if len(names) < FAST_PATH_MAX_NODES:
        return "fast-path"
    if num_devices == 1:
        return "single-device"
    return None


class JitFunction:
    """Lazily compiled step (``mjit``): compiled on first call per input signature."""

    def __init__(self, fn, *, mesh=None, in_shardings=None, out_shardings=None, donate_argnums=(),
                 static_argnums=(), backend=None):
        self.fn = fn
        self.mesh = mesh
        self.in_shardings = in_shardings
        self.out_shardings = out_shardings
        self.donate_argnums = donate_argnums
        self.static_argnums = static_argnums
        self.backend = backend
        self._cache: Dict[Any, Executable] = {}
        self.__name__ = getattr(fn, "__name__", "mjit")

    def _signature(self, args):
        leaves, spec = pytree.tree_flatten(args)
        sig = []
        for l in leaves:
            if isinstance(l, (torch.Tensor, ShardedTensor)):
                sig.append((tuple(l.shape), str(l.dtype)))
            else:
                sig.append(("const", repr(l)))
        return (str(spec), tuple(sig))

    def lower(self, *args) -> Executable:
        key = self._signature(args)
        if key not in self._cache:
            example = pytree.tree_map(
                lambda l: torch.empty(l.shape, dtype=l.dtype, device="meta") if isinstance(l, ShardedTensor) else l, args,
                is_leaf=lambda x: isinstance(x, ShardedTensor))
            self._cache[key] = compile_function(self.fn, example, mesh=self.mesh, donate_argnums=self.donate_argnums,
                                                backend=self.backend, in_shardings=self.in_shardings, name=self.__name__)
        return self._cache[key]

    def __call__(self, *args):
        if state.flags.ignore_transforms:
            return self.fn(*args)
        return self.lower(*args)(*args)
