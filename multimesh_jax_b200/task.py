"""Tasks, submeshes and microbatching: the user-facing MPMD API.

Same names and semantics as the reference's ``multimesh/jax/task.py``
(``TaskMesh`` :61-111, ``Task`` :114-139, ``Context`` :142-310, ``MultiMesh``
:313-539, ``parallelize`` :580-699, ``task`` :836-910, ``microbatch`` :913-1149)
re-expressed for PyTorch: a step function is captured once with ``torch.fx``;
while it is being captured the functions below tag the operators that are
created (forward *and* backward) with the task / scope / loop they belong to.
Outside a capture (or under ``ignore_transforms()``) ``task`` and
``microbatch`` are the identity, so the same model code runs un-partitioned.
"""
from __future__ import annotations

import contextlib
import re
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple, Union

import torch
from torch.utils import _pytree as pytree

from . import state

# ----------------------------------------------------------------------------
# Submesh descriptors
# ----------------------------------------------------------------------------


class TaskMesh:
    """A submesh: device ordinals (relative to the executable's device list),
    axis sizes and axis names. Only contiguous device ranges are supported
    (as in the reference, ``src/pjrt_client/mpmd_utils.cc:144-176``)."""

    def __init__(self, axis_sizes: Sequence[int], axis_names: Sequence[str],
                 devices: Optional[Sequence[int]] = None):
        self.axis_sizes = tuple(int(s) for s in axis_sizes)
        self.axis_names = tuple(axis_names)
        if len(self.axis_sizes) != len(self.axis_names):
            raise ValueError("axis_sizes and axis_names must have the same length")
        n = 1
        for s in self.axis_sizes:
            n *= s
        if devices is None:
            devices = list(range(n))
        self.devices = [int(d) for d in devices]
        if len(self.devices) != n:
            raise ValueError(f"mesh of shape {self.axis_sizes} needs {n} devices, got {len(self.devices)}")
        if any(b - a != 1 for a, b in zip(self.devices, self.devices[1:])):
            raise ValueError("submesh devices must be a contiguous ascending range")

    @property
    def size(self) -> int:
        return len(self.devices)

    @property
    def shape(self) -> Dict[str, int]:
        return dict(zip(self.axis_names, self.axis_sizes))

    def place(self, devices: Sequence[int]) -> "TaskMesh":
        """Same mesh shape on other devices."""
        return TaskMesh(self.axis_sizes, self.axis_names, devices)

    @property
    def abstract_mesh(self) -> Dict[str, int]:
        """Axis names and sizes without the devices (multimesh/jax/task.py:108-110)."""
        return self.shape

    def __eq__(self, other):
        return (isinstance(other, TaskMesh) and self.axis_sizes == other.axis_sizes
                and self.axis_names == other.axis_names and self.devices == other.devices)

    def __hash__(self):
        return hash((self.axis_sizes, self.axis_names, tuple(self.devices)))

    def __repr__(self):
        return f"TaskMesh({dict(zip(self.axis_names, self.axis_sizes))}, devices=[{self.devices[0]}..{self.devices[-1]}])"


@dataclass
class Task:
    """Per-task options.

    ``logical_axes`` is a priority-ordered list of ``(logical name, mesh axis)``.
    Exactly one of ``mesh`` / ``mesh_slice`` is given for regex-registered
    tasks; ``mesh_slice`` selects indices along axes of the enclosing
    :class:`MultiMesh`. ``split_backprop=(critical_suffix, noncritical_suffix)``
    asks the compiler to split the backward task into activation-gradient and
    weight-gradient halves (needed by the zero-bubble schedule).
    ``loop_dependent_mesh_slice(i)`` returns the mesh slice used by microbatch ``i``.
    """
    name: Optional[str] = None
    mesh: Optional[TaskMesh] = None
    logical_axes: Sequence[Tuple[str, str]] = ()
    mesh_slice: Optional[Dict[str, int]] = None
    extra_axes: Sequence[str] = ()
    split_backprop: Optional[Tuple[str, str]] = None
    loop_dependent_mesh_slice: Optional[Callable[[int], Dict[str, int]]] = None


TaskFactory = Callable[[str, bool], Task]


@dataclass
class _Registration:
    matcher: str
    factory: TaskFactory
    mesh: Optional["MultiMesh"] = None


class Context:
    """A scope of regex -> task registrations. Contexts nest; the innermost
    match wins (``src/pjrt_client/hlo_partition.cc:379-460``)."""

    _stack: List["Context"] = []

    def __init__(self):
        self.registrations: List[_Registration] = []

    def register_task(self, matcher: str, task: Optional[Task] = None,
                      factory: Optional[TaskFactory] = None) -> None:
        if (task is None) == (factory is None):
            raise ValueError("give exactly one of task= / factory=")
        if "(" not in matcher:
            matcher = f"({matcher})"
        re.compile(matcher)
        if factory is None:
            fixed = task

            def factory(name: str, backprop: bool, _t=fixed) -> Task:  # noqa: ARG001
                return _t
        self.registrations.append(_Registration(matcher, factory, self if isinstance(self, MultiMesh) else None))

    def __enter__(self):
        Context._stack.append(self)
        return self

    def __exit__(self, *exc):
        Context._stack.pop()
        return False

    def find_matching_slice_in_scope(self) -> Optional[Mapping[str, int]]:
        """Mesh slice of the task this context registers for the operator name stack at this point
        of a capture: innermost scope first, and within a scope the registration made last. ``None``
        outside a capture or when nothing matches; an error when the matching task names a whole
        mesh instead of a slice (multimesh/jax/task.py:160-182)."""
        scopes = [e.name for e in state.trace.scopes] if state.trace.active else []
        for scope in reversed(scopes):
            for reg in reversed(self.registrations):
                m = re.search(reg.matcher, scope)
                if not m:
                    continue
                t = reg.factory(m.group(1), False)
                if t.mesh_slice is None:
                    raise ValueError(f"task {m.group(1)} does not return a mesh slice: {t}")
                return t.mesh_slice
        return None

    @staticmethod
    def active_registrations() -> List[_Registration]:
        """Innermost context first."""
        out: List[_Registration] = []
        for ctx in reversed(Context._stack):
            out.extend(reversed(ctx.registrations))
        out.extend(reversed(_global_context.registrations))
        return out


_global_context = Context()


def register_task(matcher: str, task: Optional[Task] = None, factory: Optional[TaskFactory] = None) -> None:
    """Registers a regex task in the innermost active context (or globally)."""
    ctx = Context._stack[-1] if Context._stack else _global_context
    ctx.register_task(matcher, task=task, factory=factory)


def clear_tasks() -> None:
    """Drops every global registration (``multimesh_jax_impl.cc`` ``clear_tasks``)."""
    _global_context.registrations.clear()


class MultiMesh(Context):
    """The global device mesh plus a registration context.

    ``MultiMesh((2, 4), ("stage", "model"))`` describes 8 devices; ``slice(stage=1)``
    returns the :class:`TaskMesh` of devices 4..7 with the remaining axis
    ``model``. Entering the mesh turns on ``autoshard`` so that
    ``with_sharding_constraint`` records logical axis names."""

    _current: List["MultiMesh"] = []

    def __init__(self, axis_sizes: Sequence[int], axis_names: Sequence[str],
                 devices: Optional[Sequence[int]] = None):
        super().__init__()
        self.mesh = TaskMesh(axis_sizes, axis_names, devices)
        self._autoshard_cm = None

    # duck-typed mesh properties
    @property
    def axis_names(self):
        return self.mesh.axis_names

    @property
    def axis_sizes(self):
        return self.mesh.axis_sizes

    @property
    def devices(self):
        return self.mesh.devices

    @property
    def shape(self):
        return self.mesh.shape

    @property
    def size(self):
        return self.mesh.size

    @property
    def shape_tuple(self) -> Tuple[Tuple[str, int], ...]:
        return tuple(zip(self.mesh.axis_names, self.mesh.axis_sizes))

    @property
    def abstract_mesh(self) -> Dict[str, int]:
        return self.mesh.abstract_mesh

    @property
    def empty(self) -> bool:
        return self.mesh.size == 0

    @property
    def local_devices(self) -> List[int]:
        """Device ordinals of the mesh that this process drives: all of them in a one-process job,
        the rank's own one in a one-process-per-GPU job (``torch.distributed`` initialised)."""
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            return [d for d in self.mesh.devices if d == dist.get_rank()]
        return list(self.mesh.devices)

    @property
    def is_multi_process(self) -> bool:
        return len(self.local_devices) != self.mesh.size

    def single_slice_devices(self, **axis_idx: int):
        """The device ordinals with the named axes fixed, as a nested list that keeps every axis of
        the mesh (fixed axes have extent 1). Unlike :meth:`slice` the result need not be a contiguous
        range: this is a query, not a task placement (multimesh/jax/task.py:383-390)."""
        names, sizes = self.mesh.axis_names, self.mesh.axis_sizes
        for a in axis_idx:
            if a not in names:
                raise ValueError(f"unknown mesh axis {a!r}")

        def build(axis: int, flat: int):
            if axis == len(sizes):
                return self.mesh.devices[flat]
            picks = [axis_idx[names[axis]]] if names[axis] in axis_idx else range(sizes[axis])
            return [build(axis + 1, flat * sizes[axis] + i) for i in picks]
        return build(0, 0)

    def single_slice_ids(self, **axis_idx: int) -> List[int]:
        """Flat list of the device ordinals of :meth:`single_slice_devices`."""
        out: List[int] = []

        def walk(x):
            if isinstance(x, list):
                for y in x:
                    walk(y)
            else:
                out.append(x)
        walk(self.single_slice_devices(**axis_idx))
        return out

    def slice(self, **axis_idx: int) -> TaskMesh:
        """Sub-mesh with the named axes fixed at the given indices. The result
        must be a contiguous device range, i.e. sliced axes must be leading axes
        (or all preceding axes have size 1)."""
        names, sizes = self.mesh.axis_names, self.mesh.axis_sizes
        for a in axis_idx:
            if a not in names:
                raise ValueError(f"unknown mesh axis {a!r}")
        strides = []
        acc = 1
        for s in reversed(sizes):
            strides.append(acc)
            acc *= s
        strides = list(reversed(strides))
        devs = []
        for flat in range(self.mesh.size):
            coord = [(flat // st) % sz for st, sz in zip(strides, sizes)]
            if all(coord[names.index(a)] == i for a, i in axis_idx.items()):
                devs.append(self.mesh.devices[flat])
        keep = [(n, s) for n, s in zip(names, sizes) if n not in axis_idx]
        if not keep:
            keep = [("x", 1)]
        return TaskMesh([s for _, s in keep], [n for n, _ in keep], devs)

    def __enter__(self):
        super().__enter__()
        MultiMesh._current.append(self)
        from . import lib
        self._autoshard_cm = lib.autoshard(True)
        self._autoshard_cm.__enter__()
        return self

    def __exit__(self, *exc):
        self._autoshard_cm.__exit__(*exc)
        MultiMesh._current.pop()
        return super().__exit__(*exc)

    @staticmethod
    def current() -> Optional["MultiMesh"]:
        return MultiMesh._current[-1] if MultiMesh._current else None

    def __repr__(self):
        return f"MultiMesh({self.mesh.shape})"


def get_global_mesh() -> TaskMesh:
    """The whole mesh of the innermost active :class:`MultiMesh` (``with mesh:``), devices included
    (multimesh/jax/task.py:1152-1153: the physical mesh of the enclosing mesh context)."""
    mesh = MultiMesh.current()
    if mesh is None:
        raise RuntimeError("get_global_mesh() needs an active MultiMesh")
    return mesh.mesh


def get_abstract_global_mesh() -> Dict[str, int]:
    """Axis names and sizes of the active mesh without its devices: what sharding rules and
    shape-only code may depend on (multimesh/jax/task.py:1156-1157)."""
    return dict(get_global_mesh().shape)


def slice_global_mesh(**axis_idx: int) -> TaskMesh:
    mesh = MultiMesh.current()
    if mesh is None:
        raise RuntimeError("slice_global_mesh() needs an active MultiMesh")
    return mesh.slice(**axis_idx)


# ----------------------------------------------------------------------------
# Task payloads handed to the graph compiler
# ----------------------------------------------------------------------------


def resolve_task_mesh(t: Task, enclosing: Optional[MultiMesh], microbatch: Optional[int] = None) -> TaskMesh:
    if microbatch is not None and t.loop_dependent_mesh_slice is not None:
        if enclosing is None:
            raise ValueError("loop_dependent_mesh_slice needs a MultiMesh")
        return enclosing.slice(**t.loop_dependent_mesh_slice(microbatch))
    if (t.mesh is None) == (t.mesh_slice is None):
        raise ValueError("a Task needs exactly one of mesh / mesh_slice")
    if t.mesh is not None:
        return t.mesh
    if enclosing is None:
        raise ValueError("mesh_slice needs an enclosing MultiMesh")
    return enclosing.slice(**t.mesh_slice)


def task_payload(t: Task, name: str, enclosing: Optional[MultiMesh], num_microbatches: int = 0) -> Dict[str, Any]:
    """The 7-field record the compiler receives for one task
    (``src/pjrt_client/pycallback_types.h:12-28``)."""
    mesh = resolve_task_mesh(t, enclosing)
    loop_devices: List[List[int]] = []
    if t.loop_dependent_mesh_slice is not None:
        for i in range(max(num_microbatches, 1)):
            m = resolve_task_mesh(t, enclosing, microbatch=i)
            if m.size != mesh.size:
                raise ValueError("loop_dependent_mesh_slice must keep the device count")
            loop_devices.append(list(m.devices))
    return {
        "name": t.name or name,
        "devices": list(mesh.devices),
        "dims": list(mesh.axis_sizes),
        "device_axes": list(mesh.axis_names),
        "logical_axes": [[a, b] for a, b in t.logical_axes],
        "split_backprop": list(t.split_backprop) if t.split_backprop else [],
        "loop_dependent_devices": loop_devices,
    }


# ----------------------------------------------------------------------------
# Trace-time scopes
# ----------------------------------------------------------------------------


@contextlib.contextmanager
def named_scope(name: str):
    """Adds ``name`` to the operator name stack (the analogue of
    ``jax.named_scope``); regex tasks match against the joined stack."""
    if not state.trace.active:
        yield
        return
    state.trace.scopes.append(state.ScopeEntry(name))
    try:
        yield
    finally:
        state.trace.scopes.pop()


@contextlib.contextmanager
def module_scopes(module: torch.nn.Module):
    """While active, every sub-module's forward runs inside a scope named by
    its qualified name, so regex tasks can match module paths."""
    handles = []
    for qual, sub in module.named_modules():
        if not qual:
            continue

        def pre(_m, _args, _q=qual):
            if state.trace.active:
                state.trace.scopes.append(state.ScopeEntry(_q))

        def post(_m, _args, _out, _q=qual):
            if state.trace.active and state.trace.scopes and state.trace.scopes[-1].name == _q:
                state.trace.scopes.pop()

        handles.append(sub.register_forward_pre_hook(pre))
        handles.append(sub.register_forward_hook(post, always_call=True))
    try:
        yield
    finally:
        for h in handles:
            h.remove()


def _transforms_active() -> bool:
    return state.trace.active and not state.flags.ignore_transforms


def task(fun: Optional[Callable] = None, *, name: Optional[str] = None, mesh: Optional[TaskMesh] = None,
         devices: Optional[Sequence[int]] = None, logical_axes: Sequence[Tuple[str, str]] = (),
         split_backprop: Optional[Tuple[str, str]] = None):
    """Marks ``fun`` as an explicit task. All operators created while it runs
    belong to the task; operators of its backward pass form a separate task
    ``<name>_bwd`` on the same devices (``multimesh/jax/task.py:797-833``).
    Default placement: every device, one mesh axis ``x``."""
    if fun is None:
        return lambda f: task(f, name=name, mesh=mesh, devices=devices, logical_axes=logical_axes,
                              split_backprop=split_backprop)
    base = name or getattr(fun, "__name__", "task")

    def wrapped(*args, **kwargs):
        if not _transforms_active():
            return fun(*args, **kwargs)
        m = mesh
        if m is None and devices is not None:
            m = TaskMesh((len(devices),), ("x",), devices)
        payload = {"name": base, "devices": list(m.devices) if m else [],
                   "dims": list(m.axis_sizes) if m else [],
                   "device_axes": list(m.axis_names) if m else ["x"],
                   "logical_axes": [[a, b] for a, b in logical_axes],
                   "split_backprop": list(split_backprop) if split_backprop else [],
                   "loop_dependent_devices": []}
        state.trace.scopes.append(state.ScopeEntry("", explicit_task=payload))
        try:
            return fun(*args, **kwargs)
        finally:
            state.trace.scopes.pop()

    wrapped.__name__ = base
    wrapped.__wrapped__ = fun
    return wrapped


# ----------------------------------------------------------------------------
# Microbatching
# ----------------------------------------------------------------------------

_mm_lib = torch.library.Library("mm", "FRAGMENT")
_mm_lib.define("microbatch_slice(Tensor x, int dim, int size, int loop) -> Tensor")
_mm_lib.define("microbatch_out(Tensor y, int loop, str dtype) -> Tensor")


def _mb_slice_impl(x, dim, size, loop):
    return x.narrow(dim, 0, size).clone()


def _acc_dtype(y, dtype: str):
    if dtype and y.is_floating_point():
        return getattr(torch, dtype)
    return y.dtype


def _mb_out_impl(y, loop, dtype):
    return y.to(_acc_dtype(y, dtype), copy=True)


torch.library.impl(_mm_lib, "microbatch_slice", "CompositeExplicitAutograd")(_mb_slice_impl)
torch.library.impl(_mm_lib, "microbatch_out", "CompositeExplicitAutograd")(_mb_out_impl)
torch.library.register_fake("mm::microbatch_slice")(lambda x, dim, size, loop: x.narrow(dim, 0, size).clone())
torch.library.register_fake("mm::microbatch_out")(
    lambda y, loop, dtype: torch.empty_like(y, dtype=_acc_dtype(y, dtype)))

SCHEDULES = ("gpipe", "1f1b", "wavefront", "custom", "zero-bubble-h2", "prefetch-wavefront")


def _canonical_custom_schedule(custom, num_microbatches: int):
    """Rows = meshes; entries ``task`` or ``(microbatch, task)``. Bare task
    names get their occurrence count as the microbatch index; every name must
    occur exactly ``num_microbatches`` times (``multimesh/jax/task.py:1050-1069``)."""
    out = []
    counts: Dict[str, int] = {}
    for row in custom:
        new_row = []
        for entry in row:
            if isinstance(entry, str):
                idx = counts.get(entry, 0)
                tname = entry
            else:
                idx, tname = entry
            counts[tname] = counts.get(tname, 0) + 1
            new_row.append([int(idx), tname])
        out.append(new_row)
    for tname, c in counts.items():
        if c != num_microbatches:
            raise ValueError(f"custom schedule: task {tname!r} appears {c} times, expected {num_microbatches}")
    return out


def microbatch(fun: Callable, *, dim: int = 0, size: int, argnum: Union[int, Sequence[int]] = 0,
               schedule: Optional[str] = None, custom_schedule=None, interleave: Optional[int] = None,
               unrolling: Optional[int] = None, num_stages: Optional[int] = None,
               batch_dim: Optional[int] = None, accumulate_dtype: Optional[torch.dtype] = None):
    """Runs ``fun`` once per microbatch of ``size`` rows (argument ``argnum``
    sliced along ``dim``) and **sums** every output over the microbatches.
    ``schedule`` is one of ``gpipe``, ``1f1b``/``wavefront``, ``prefetch-wavefront``,
    ``zero-bubble-h2`` or ``custom``. With a single microbatch, outside a capture,
    or under ``ignore_transforms`` ``fun`` is called directly on the whole batch."""
    if schedule is not None and schedule not in SCHEDULES:
        raise ValueError(f"unknown schedule {schedule!r}; expected one of {SCHEDULES}")
    argnums = (argnum,) if isinstance(argnum, int) else tuple(argnum)

    def wrapped(*args, **kwargs):
        if not _transforms_active():
            return fun(*args, **kwargs)
        leaves = []
        for a in argnums:
            leaves.extend(l for l in pytree.tree_leaves(args[a]) if isinstance(l, torch.Tensor))
        if not leaves:
            raise ValueError("microbatch: no tensor found in the microbatched argument")
        total = leaves[0].shape[dim]
        if any(l.shape[dim] != total for l in leaves):
            raise ValueError("microbatch: all sliced leaves must share the size of the sliced dimension")
        if total % size:
            raise ValueError(f"microbatch: dimension {total} is not divisible by size {size}")
        n = total // size
        if n == 1:
            return fun(*args, **kwargs)
        tr = state.trace
        if tr.loop is not None:
            raise NotImplementedError("nested microbatch loops are not supported")
        cfg: Dict[str, Any] = {"num_microbatches": n, "slice_dim": dim, "size": size,
                               "batch_dim": dim if batch_dim is None else batch_dim}
        for key, val in (("interleave", interleave), ("unrolling", unrolling), ("num_stages", num_stages),
                         ("schedule", schedule)):
            if val is not None:
                cfg[key] = val
        if custom_schedule is not None:
            cfg["custom_schedule"] = _canonical_custom_schedule(custom_schedule, n)
        if accumulate_dtype is not None:
            cfg["accumulate_dtype"] = str(accumulate_dtype).replace("torch.", "")
        loop_id = len(tr.loop_configs)
        cfg["id"] = loop_id
        tr.loop_configs.append(cfg)
        tr.loop = cfg
        try:
            new_args = list(args)
            for a in argnums:
                new_args[a] = pytree.tree_map(
                    lambda x: torch.ops.mm.microbatch_slice(x, dim, size, loop_id)
                    if isinstance(x, torch.Tensor) else x, args[a])
            out = fun(*new_args, **kwargs)
            acc_name = cfg.get("accumulate_dtype", "")
            out = pytree.tree_map(
                lambda y: torch.ops.mm.microbatch_out(y, loop_id, acc_name) if isinstance(y, torch.Tensor) else y,
                out)
        finally:
            tr.loop = None
        return out

    wrapped.__name__ = getattr(fun, "__name__", "microbatched")
    return wrapped


# ----------------------------------------------------------------------------
# Differentiation helper
# ----------------------------------------------------------------------------


def value_and_grad(fun: Callable, argnums: Union[int, Sequence[int]] = 0, has_aux: bool = False):
    """``jax.value_and_grad`` for PyTorch: returns ``(value, grads)`` where
    ``grads`` mirrors the structure of the differentiated argument(s). The
    backward pass runs inside the call, so under a capture its operators are
    recorded in the same graph (and tagged as the backward of their task)."""
    single = isinstance(argnums, int)
    nums = (argnums,) if single else tuple(argnums)

    def wrapped(*args, **kwargs):
        args = list(args)
        specs = []
        diff_leaves: List[torch.Tensor] = []
        for a in nums:
            leaves, spec = pytree.tree_flatten(args[a])
            new_leaves = []
            for l in leaves:
                if isinstance(l, torch.Tensor) and l.is_floating_point():
                    nl = l.detach().requires_grad_(True)
                    diff_leaves.append(nl)
                    new_leaves.append(nl)
                else:
                    new_leaves.append(l)
            args[a] = pytree.tree_unflatten(new_leaves, spec)
            specs.append((spec, new_leaves))
        with torch.enable_grad():
            out = fun(*args, **kwargs)
            value, aux = (out if has_aux else (out, None))
            grads = torch.autograd.grad(value, diff_leaves, allow_unused=True)
        grads = [g if g is not None else torch.zeros_like(l) for g, l in zip(grads, diff_leaves)]
        it = iter(grads)
        results = []
        for spec, leaves in specs:
            gl = [next(it) if (isinstance(l, torch.Tensor) and l.is_floating_point()) else None for l in leaves]
            results.append(pytree.tree_unflatten(gl, spec))
        g_out = results[0] if single else tuple(results)
        value = value.detach()
        return ((value, aux), g_out) if has_aux else (value, g_out)

    return wrapped


# ----------------------------------------------------------------------------
# Ahead-of-time compilation
# ----------------------------------------------------------------------------


def parallelize(fun: Callable, init_params: Callable[[], Any], get_input_batch: Optional[Callable[[], Any]] = None,
                *, mesh: Optional[MultiMesh] = None, donate_argnums: Sequence[int] = (), backend: Optional[str] = None):
    """Ahead-of-time compile ``fun(params, batch)``.

    Shapes are taken from ``init_params()`` / ``get_input_batch()`` evaluated on
    the meta device; the compiler chooses input shardings; the returned
    initialisers produce parameters (and a batch) already laid out that way.
    Returns ``(compiled, init_sharded_params[, init_sharded_batch])``
    (``multimesh/jax/task.py:580-699``)."""
    from . import lib
    from .compiler.api import compile_function

    with lib.autoshard(True):
        with torch.device("meta"):
            abstract_params = init_params()
            abstract_batch = get_input_batch() if get_input_batch is not None else None
        example = (abstract_params,) if abstract_batch is None else (abstract_params, abstract_batch)
        compiled = compile_function(fun, example, mesh=mesh or MultiMesh.current(),
                                    donate_argnums=donate_argnums, backend=backend)

    def init_sharded_params():
        return compiled.shard_argument(0, init_params())

    if get_input_batch is None:
        return compiled, init_sharded_params

    def init_sharded_batch():
        return compiled.shard_argument(1, get_input_batch())

    return compiled, init_sharded_params, init_sharded_batch
