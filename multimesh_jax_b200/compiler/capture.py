"""Capture of one step function with ``torch.fx`` and export to the native graph IR.

``make_fx`` records forward *and* backward operators of the step (the backward
pass runs inside the traced function through ``torch.autograd.grad``). While it
runs, every created node is tagged with the trace-time state of
:mod:`multimesh_jax_b200.state`: the name stack, the enclosing explicit task
and microbatch loop. Backward nodes inherit the tag of the forward operator
whose autograd node is executing (matched by autograd sequence number), with
``backprop=True`` - the counterpart of the reference recognising backward
instructions by ``transpose(jvp`` in JAX op names
(``src/pjrt_client/hlo_partition.cc:379-460``).
"""
from __future__ import annotations

import json
import operator
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.fx as fx
import torch.fx.proxy as fx_proxy
from torch.fx.experimental.proxy_tensor import make_fx
from torch.utils import _pytree as pytree

from .. import state
from ..task import Context, MultiMesh, task_payload

_DTYPE_NAMES = {
    torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float64: "float64",
    torch.int8: "int8", torch.int16: "int16", torch.int32: "int32", torch.int64: "int64", torch.uint8: "uint8",
    torch.bool: "bool", torch.float8_e4m3fn: "float8_e4m3fn", torch.float8_e5m2: "float8_e5m2",
}
DTYPE_FROM_NAME = {v: k for k, v in _DTYPE_NAMES.items()}


def dtype_name(dt: torch.dtype) -> str:
    return _DTYPE_NAMES[dt]


@dataclass
class Captured:
    """A captured step: the fx graph, the native graph and the maps between them."""
    gm: fx.GraphModule
    graph: Any                                  # _mm_C.Graph
    node_of_fx: Dict[fx.Node, int]              # fx node -> IR node id
    fx_of_node: Dict[int, fx.Node]              # IR node id -> fx node
    value_of_fx: Dict[Any, int]                 # (fx node, out index or None) -> IR value id
    out_index_map: Dict[int, List[Optional[int]]]  # IR node id -> for each fx result position, output slot or None
    in_spec: Any
    out_spec: Any
    num_inputs: int
    input_is_tensor: List[bool]
    constant_inputs: List[Any]
    output_values: List[int]
    output_constants: Dict[int, Any]            # flat output position -> non-tensor constant
    loop_configs: List[Dict[str, Any]] = field(default_factory=list)


class _NodeTagger:
    """Patches ``TracerBase.create_node`` for the duration of a capture."""

    def __enter__(self):
        self._orig = fx_proxy.TracerBase.create_node
        tr = state.trace
        orig = self._orig

        def create_node(tracer, kind, target, args, kwargs, name=None, type_expr=None):
            node = orig(tracer, kind, target, args, kwargs, name, type_expr)
            try:
                cur = torch._C._current_autograd_node()
            except Exception:  # pragma: no cover
                cur = None
            if cur is not None:
                tag = tr.scope_by_seq.get(cur._sequence_nr())
                if tag is None:
                    tag = dict(tr.current_tag())
                    tag["scope"] = ""
                    tag["task"] = None
                node.meta["mm"] = dict(tag, backprop=True)
            else:
                tag = tr.current_tag()
                seq = torch.autograd._get_sequence_nr() - 1
                tr.scope_by_seq.setdefault(seq, tag)
                node.meta["mm"] = dict(tag, backprop=False)
            return node

        fx_proxy.TracerBase.create_node = create_node
        return self

    def __exit__(self, *exc):
        fx_proxy.TracerBase.create_node = self._orig
        return False


def _jsonable(x):
    if isinstance(x, (bool, int, float, str)) or x is None:
        return x
    if isinstance(x, (list, tuple)):
        return [_jsonable(e) for e in x]
    if isinstance(x, torch.dtype):
        return dtype_name(x) if x in _DTYPE_NAMES else str(x)
    if isinstance(x, (torch.device, torch.layout, torch.memory_format)):
        return str(x)
    if isinstance(x, torch.SymInt):
        return int(x)
    return str(x)


def op_name(target) -> str:
    if isinstance(target, torch._ops.OpOverload):
        ns, rest = target._schema.name.split("::")
        ov = target._overloadname or "default"
        return f"{ns}.{rest}.{ov}"
    if isinstance(target, torch._ops.OpOverloadPacket):
        return str(target)
    return getattr(target, "__name__", str(target))


# Sharding rules of custom operators, registered next to the operator definitions.
SHARD_RULES: Dict[str, Callable[[fx.Node, List[Tuple[int, ...]], List[Tuple[int, ...]]], Dict[str, Any]]] = {}


def register_shard_rule(op: str):
    def deco(fn):
        SHARD_RULES[op] = fn
        return fn
    return deco


def capture(fn: Callable, example_args: Sequence[Any], *, device: Optional[torch.device] = None,
            mesh: Optional[MultiMesh] = None) -> Captured:
    """Traces ``fn(*example_args)``. Tensor leaves become graph inputs (their
    values are never read: tracing runs on fake tensors); other leaves are
    baked in as constants."""
    from .. import _mm_C
    from torch._subclasses.fake_tensor import FakeTensorMode

    flat_args, in_spec = pytree.tree_flatten(tuple(example_args))
    is_tensor = [isinstance(a, torch.Tensor) for a in flat_args]
    fake_mode = FakeTensorMode(allow_non_fake_inputs=True)
    target_device = device or torch.device("cpu")

    def to_fake(t: torch.Tensor):
        with fake_mode:
            return torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=target_device)

    tensor_inputs = [to_fake(a) for a, ok in zip(flat_args, is_tensor) if ok]
    out_info: Dict[str, Any] = {}

    def flat_fn(*tensors):
        it = iter(tensors)
        leaves = [next(it) if ok else a for a, ok in zip(flat_args, is_tensor)]
        args = pytree.tree_unflatten(leaves, in_spec)
        out = fn(*args)
        flat_out, out_spec = pytree.tree_flatten(out)
        out_info["spec"] = out_spec
        out_info["is_tensor"] = [isinstance(o, torch.Tensor) for o in flat_out]
        out_info["constants"] = {i: o for i, o in enumerate(flat_out) if not isinstance(o, torch.Tensor)}
        return [o for o in flat_out if isinstance(o, torch.Tensor)]

    tr = state.trace
    if tr.active:
        raise RuntimeError("nested captures are not supported")
    tr.reset()
    tr.active = True
    try:
        with _NodeTagger():
            gm = make_fx(flat_fn, tracing_mode="fake", _allow_non_fake_inputs=True)(*tensor_inputs)
        loop_configs = list(tr.loop_configs)
    finally:
        tr.reset()

    graph = _mm_C.Graph()
    value_of_fx: Dict[Any, int] = {}
    node_of_fx: Dict[fx.Node, int] = {}
    fx_of_node: Dict[int, fx.Node] = {}
    out_index_map: Dict[int, List[Optional[int]]] = {}
    output_values: List[int] = []
    enclosing = mesh or MultiMesh.current()
    num_mb = loop_configs[0]["num_microbatches"] if loop_configs else 0

    def tensor_value(arg) -> Optional[int]:
        if isinstance(arg, fx.Node):
            return value_of_fx.get((arg, None))
        return None

    for node in gm.graph.nodes:
        if node.op == "placeholder":
            val = node.meta["val"]
            vid = graph.add_input(node.name, list(val.shape), dtype_name(val.dtype))
            value_of_fx[(node, None)] = vid
            continue
        if node.op == "output":
            outs = node.args[0]
            for o in outs:
                output_values.append(value_of_fx[(o, None)])
            continue
        if node.op != "call_function":
            raise NotImplementedError(f"unsupported fx node kind {node.op}")
        if node.target is operator.getitem:
            src, idx = node.args
            key = (src, idx)
            if key in value_of_fx:
                value_of_fx[(node, None)] = value_of_fx[key]
            continue
        flat, _ = pytree.tree_flatten((node.args, node.kwargs))
        inputs: List[int] = []
        nontensor: List[Any] = []
        for a in flat:
            v = tensor_value(a)
            if v is not None:
                inputs.append(v)
        for a in node.args:
            if isinstance(a, fx.Node) and tensor_value(a) is not None:
                continue
            if isinstance(a, (list, tuple)) and any(isinstance(e, fx.Node) for e in a):
                continue
            nontensor.append(_jsonable(a))
        val = node.meta.get("val")
        if isinstance(val, torch.Tensor):
            vals = [val]
            slots: List[Optional[int]] = [0]
            single = True
        elif isinstance(val, (list, tuple)):
            vals, slots = [], []
            for e in val:
                if isinstance(e, torch.Tensor):
                    slots.append(len(vals))
                    vals.append(e)
                else:
                    slots.append(None)
            single = False
        else:
            # no tensor result (e.g. a symbolic size): nothing to export
            continue
        name = op_name(node.target)
        tag = node.meta.get("mm", {"scope": "", "task": None, "loop": -1, "backprop": False})
        attrs = {"args": json.dumps(nontensor), "fx": node.name}
        rule = SHARD_RULES.get(name)
        if rule is not None:
            in_shapes = [tuple(graph.value(v)["shape"]) for v in inputs]
            attrs["shard_rule"] = json.dumps(rule(node, in_shapes, [tuple(v.shape) for v in vals]))
        explicit = ""
        if tag.get("task") is not None:
            explicit = json.dumps(tag["task"])
        nid, outs = graph.add_node(name, inputs, [list(v.shape) for v in vals], [dtype_name(v.dtype) for v in vals],
                                   attrs, tag.get("scope", ""), bool(tag.get("backprop")), int(tag.get("loop", -1)),
                                   explicit, "")
        node_of_fx[node] = nid
        fx_of_node[nid] = node
        out_index_map[nid] = slots
        if single:
            value_of_fx[(node, None)] = outs[0]
        else:
            for pos, slot in enumerate(slots):
                if slot is not None:
                    value_of_fx[(node, pos)] = outs[slot]
    graph.set_outputs(output_values)
    for cfg in loop_configs:
        graph.add_loop(json.dumps(cfg))

    return Captured(gm=gm, graph=graph, node_of_fx=node_of_fx, fx_of_node=fx_of_node, value_of_fx=value_of_fx,
                    out_index_map=out_index_map, in_spec=in_spec, out_spec=out_info["spec"],
                    num_inputs=len(tensor_inputs), input_is_tensor=is_tensor,
                    constant_inputs=[a for a, ok in zip(flat_args, is_tensor) if not ok],
                    output_values=output_values, output_constants=out_info["constants"],
                    loop_configs=loop_configs)


def make_partition(num_devices: int, mesh: Optional[MultiMesh], num_microbatches: int = 0):
    """Creates the native colour table and registers the active regex contexts."""
    from .. import _mm_C

    part = _mm_C.Partition(0, num_devices)
    for reg in Context.active_registrations():
        enclosing = reg.mesh or mesh

        def cb(matched: str, backprop: bool, _reg=reg, _mesh=enclosing) -> str:
            t = _reg.factory(matched, backprop)
            return json.dumps(task_payload(t, "", _mesh, num_microbatches))

        part.register_task_factory(reg.matcher, cb)
    return part
