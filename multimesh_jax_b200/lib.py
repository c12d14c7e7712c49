"""Context managers, sharding annotations and ``mjit``.

Counterpart of the reference's ``multimesh/jax/lib.py``: ``ignore_transforms``
(:50-74), ``enable_fast_path`` (:77-94), ``enable_recomputation`` (:97-115),
``autoshard`` (:118-132), ``with_sharding_constraint`` (:144-230), ``tasks``
/ ``context`` (:255-310) and ``mjit`` (:313-351).
"""
from __future__ import annotations

import contextlib
from typing import Any, Callable, Dict, Optional, Sequence, Tuple, Union

import torch

from . import no_op as _no_op
from . import state
from .task import Context, MultiMesh, Task

_auto_sharding = _no_op.no_op(_no_op.AUTO_SHARDING)


def ignore_transforms(enabled: bool = True):
    """Debug aid: ``task`` / ``microbatch`` / sharding annotations become no-ops."""
    return state._flag("ignore_transforms", enabled)


def should_ignore_transforms() -> bool:
    return state.flags.ignore_transforms or not state.trace.active


def enable_fast_path(enabled: bool = True):
    """Small single-task programs bypass the MPMD runtime when enabled."""
    return state._flag("fast_path", enabled)


def enable_recomputation(enabled: bool = True):
    """Allows the compiler to recompute cheap producer trees in the consumer
    task instead of sending their result across submeshes."""
    return state._flag("recomputation", enabled)


def autoshard(enabled: bool = True):
    """In autoshard mode ``with_sharding_constraint`` records *logical* axis
    names and the compiler maps them to mesh axes per task."""
    return state._flag("autoshard", enabled)


def replicate_parameters_smaller_than_num_elements(n: int) -> None:
    state.knobs["replicated_parameter_num_elements_cutoff"] = int(n)


def recompute_from_arguments_if_cost_less_than(cost: int) -> None:
    state.knobs["recompute_from_arguments_if_cost_less_than"] = int(cost)


AxisSpec = Union[None, str, Sequence[str]]


def _canonical_axes(spec: Sequence[AxisSpec], ndim: int):
    """``None`` -> [], ``"a"`` -> ["a"], trailing dims padded with []."""
    if len(spec) > ndim:
        raise ValueError(f"sharding spec {spec} has more entries than the tensor has dims ({ndim})")
    axes = []
    for s in spec:
        if s is None:
            axes.append([])
        elif isinstance(s, str):
            axes.append([s])
        else:
            axes.append([str(x) for x in s])
    axes.extend([] for _ in range(ndim - len(axes)))
    return axes


def with_sharding_constraint(x: Any, spec: Sequence[AxisSpec]):
    """Annotates ``x`` (a tensor or a pytree of tensors) with one tuple of axis
    names per dimension. In autoshard mode the names are logical and resolved
    per task through ``Task.logical_axes``; otherwise they are mesh axis names
    and fix the physical sharding directly."""
    if should_ignore_transforms():
        return x
    from torch.utils import _pytree as pytree

    def one(t):
        if not isinstance(t, torch.Tensor):
            return t
        payload = {"axes": _canonical_axes(spec, t.dim()), "logical": bool(state.flags.autoshard)}
        return _auto_sharding(t, payload)

    return pytree.tree_map(one, x)


def relayout(x: Any, spec: Sequence[AxisSpec], grad_spec: Optional[Sequence[AxisSpec]] = None):
    """A layout change point: the result equals ``x`` but is laid out as ``spec`` says (same
    conventions as :func:`with_sharding_constraint`; all ``None`` = replicated), while ``x``
    itself keeps the layout it has. Where the two differ the compiled task gathers or slices
    at this point. Typical use: parameters stored sharded over the data-parallel ranks
    (``with_sharding_constraint(w, (..., "fsdp"))``) and gathered once per step before the
    microbatch loop (``relayout(w, (..., None))``).

    ``grad_spec`` gives the layout of the cotangent that flows back through this point (the
    layout ``x`` has, normally): the backward pass then changes layout at the mirrored point,
    e.g. the all-gather of a sequence-sharded activation in front of a tensor-parallel
    projection turns into the reduce-scatter of that activation's gradient."""
    if should_ignore_transforms():
        return x
    from torch.utils import _pytree as pytree
    import json as _json

    def one(t):
        if not isinstance(t, torch.Tensor):
            return t
        payload = {"axes": _canonical_axes(spec, t.dim()), "logical": bool(state.flags.autoshard)}
        if grad_spec is not None:
            payload["grad_axes"] = _canonical_axes(grad_spec, t.dim())
        return torch.ops.mm.marker(t, "Relayout", _json.dumps(payload))

    return pytree.tree_map(one, x)


def index_class(members: Sequence[Tuple[int, int]], *, reduced_outputs: Sequence[int] = (), no_shard: bool = False,
                shares_axes: bool = False) -> Dict[str, Any]:
    """One index class of a sharding rule: the (slot, dimension) pairs that are indexed by the
    same loop variable of the operator. Slots count the tensor operands first, then the results.
    ``reduced_outputs`` lists result slots that become partial sums when the class is sharded
    (a contraction), ``no_shard`` forbids sharding the class, ``shares_axes`` lets the class use
    mesh axes that another class of the same operator already uses (expert dimension next to the
    token dimension)."""
    out = {"members": [list(m) for m in members], "no_shard": bool(no_shard),
           "reduced_outputs": [int(r) for r in reduced_outputs]}
    if shares_axes:
        out["shares_axes"] = True
    return out


def custom_partitioning(op: Any, rule: Optional[Callable] = None):
    """Gives a user-defined operator (a ``torch.library`` operator, or its ``namespace.name.overload``
    string) its sharding rule, so that the compiler shards it inside whichever task it lands in,
    on that task's own sub-mesh. ``rule(node, in_ranks, out_ranks)`` receives the graph node and the
    shapes of the tensor operands / results and returns ``{"classes": [index_class(...), ...]}``.
    Usable as a decorator. Counterpart of ``multimesh.jax.custom_partitioning``
    (multimesh/jax/task.py:542-560), which re-routes JAX's partitioner callback to the task mesh;
    here the rule is consumed by the C++ propagation pass directly."""
    from .compiler.capture import op_name, register_shard_rule
    name = op if isinstance(op, str) else op_name(op if isinstance(op, torch._ops.OpOverload) else op.default)
    if rule is None:
        return register_shard_rule(name)
    register_shard_rule(name)(rule)
    return rule


def shard_map(fun: Callable, in_specs: Sequence[Optional[Sequence[AxisSpec]]],
              out_specs: Union[Sequence[AxisSpec], Sequence[Optional[Sequence[AxisSpec]]], None] = None) -> Callable:
    """Runs ``fun`` with its arguments and results laid out as the specs say, on the sub-mesh of
    the task the call lands in (``multimesh.jax.shard_map``, multimesh/jax/task.py:562-577, does the
    same re-routing for JAX's ``shard_map``). ``in_specs`` has one entry per positional argument
    and ``out_specs`` one per result (or a single spec for a single result); an entry is a
    per-dimension tuple of mesh axis names as in :func:`with_sharding_constraint`, or None to leave
    that value to the propagation pass. ``fun`` is written over the global shapes and must be
    shard-wise (every operator in it carries a sharding rule, so it is): the compiled task then
    executes it on local tiles only, with the collectives the layouts imply. Outside a capture,
    and under :func:`ignore_transforms`, the wrapper calls ``fun`` unchanged."""
    def wrapped(*args):
        if should_ignore_transforms():
            return fun(*args)
        if len(in_specs) != len(args):
            raise ValueError(f"shard_map: {len(in_specs)} in_specs for {len(args)} arguments")
        with autoshard(False):                 # the specs name mesh axes, not logical axes
            pinned = [a if sp is None else with_sharding_constraint(a, sp) for a, sp in zip(args, in_specs)]
            out = fun(*pinned)
            if out_specs is None:
                return out
            if isinstance(out, (tuple, list)):
                specs = list(out_specs)
                if len(specs) != len(out):
                    raise ValueError(f"shard_map: {len(specs)} out_specs for {len(out)} results")
                return type(out)(o if sp is None else with_sharding_constraint(o, sp) for o, sp in zip(out, specs))
            return with_sharding_constraint(out, out_specs)
    wrapped.__name__ = getattr(fun, "__name__", "shard_map")
    return wrapped


def optional_kwargs(**kwargs):
    """The keyword arguments whose value is not ``None``: lets a caller forward only the options a
    user actually set (multimesh/jax/lib.py:247-252)."""
    return {k: v for k, v in kwargs.items() if v is not None}


@contextlib.contextmanager
def tasks(configurable: Any):
    """Registers every ``(matcher, Task | factory)`` pair produced by
    ``configurable`` (an iterable, a mapping or a zero-argument callable) for
    the duration of the block."""
    items = configurable() if callable(configurable) else configurable
    if isinstance(items, dict):
        items = items.items()
    ctx = Context()
    for matcher, t in items:
        if isinstance(t, Task):
            ctx.register_task(matcher, task=t)
        else:
            ctx.register_task(matcher, factory=t)
    with ctx:
        yield ctx


@contextlib.contextmanager
def context(*managers):
    """Enters several context managers at once."""
    with contextlib.ExitStack() as stack:
        for m in managers:
            stack.enter_context(m)
        yield


def mjit(fun: Callable, *, mesh: Optional[MultiMesh] = None, in_shardings: Any = None,
         out_shardings: Any = None, donate_argnums: Sequence[int] = (), static_argnums: Sequence[int] = (),
         backend: Optional[str] = None):
    """Just-in-time MPMD compilation: the function is captured and compiled on
    first call for the given argument shapes; ``in_shardings`` / ``out_shardings``
    are pytrees of per-dimension axis-name tuples (or ``None`` for "compiler's choice")."""
    from .compiler.api import JitFunction
    return JitFunction(fun, mesh=mesh, in_shardings=in_shardings, out_shardings=out_shardings,
                       donate_argnums=tuple(donate_argnums), static_argnums=tuple(static_argnums),
                       backend=backend)
