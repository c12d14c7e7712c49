"""Lowering of task templates to executable programs.

Each task template of the plan (a list of IR node ids) becomes a
:class:`TemplateProgram`: a flat instruction list interpreted per launch. Nodes
that came from the fx capture call their original operator (custom ``mm_ops``
operators dispatch to the hand-written CUDA kernels on CUDA tensors); nodes
created by the compiler (``mm.copy``, ``mm.dynamic_slice``, ``mm.all_reduce``,
``mm.spmd_reshard``, ``mm.accumulate``) are implemented here. One program is
built per unique task and shared by all of its microbatch instances - the
analogue of the reference compiling each unique task body once
(``src/pjrt_client/executable_cache.cc:14-28``).
"""
from __future__ import annotations

import json
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.fx as fx

from .capture import Captured, DTYPE_FROM_NAME

_SIZE_ARG_OPS = {
    "aten.view.default", "aten.reshape.default", "aten._unsafe_view.default", "aten.expand.default",
    "aten.new_zeros.default", "aten.new_empty.default", "aten.new_ones.default", "aten.new_full.default",
    "aten.zeros.default", "aten.ones.default", "aten.empty.memory_format", "aten.full.default",
    "aten.broadcast_to.default",
}


class _V:
    """Placeholder for an IR value inside an argument structure."""
    __slots__ = ("vid",)

    def __init__(self, vid: int):
        self.vid = vid


class _Dev:
    """Placeholder for 'the device this task runs on'."""


def _materialize(spec, env, ctx):
    if isinstance(spec, _V):
        return env[spec.vid]
    if isinstance(spec, _Dev):
        return ctx.torch_device
    if isinstance(spec, tuple):
        return tuple(_materialize(s, env, ctx) for s in spec)
    if isinstance(spec, list):
        return [_materialize(s, env, ctx) for s in spec]
    if isinstance(spec, dict):
        return {k: _materialize(v, env, ctx) for k, v in spec.items()}
    return spec


def _has_placeholder(spec) -> bool:
    if isinstance(spec, (_V, _Dev)):
        return True
    if isinstance(spec, (tuple, list)):
        return any(_has_placeholder(s) for s in spec)
    if isinstance(spec, dict):
        return any(_has_placeholder(v) for v in spec.values())
    return False


class Instr:
    __slots__ = ("kind", "fn", "args", "kwargs", "outs", "slots", "node_id", "extra", "static")

    def __init__(self, kind, fn, args, kwargs, outs, slots, node_id, extra=None):
        self.kind = kind
        self.fn = fn
        self.args = args
        self.kwargs = kwargs
        self.outs = outs
        self.slots = slots
        self.node_id = node_id
        self.extra = extra
        self.static = not (_has_placeholder(args) or _has_placeholder(kwargs))


class TemplateProgram:
    def __init__(self, template: dict, instrs: List[Instr], inputs: List[int], outputs: List[int],
                 last_use: Dict[int, int]):
        self.template = template
        self.instrs = instrs
        self.inputs = inputs
        self.outputs = outputs
        self.name = template["name"]
        self.mesh_dims = template["mesh_dims"]
        self.device_start = template["device_start"]
        self._last_use = last_use
        self.fused_acc: Dict[int, bool] = {}

    def run(self, ctx, scalars: Sequence[int], inputs: Sequence[torch.Tensor],
            acc_bufs: Optional[Sequence[Optional[torch.Tensor]]] = None) -> List[torch.Tensor]:
        """``acc_bufs[k]`` is the current accumulator tile of output ``k`` (or None for its
        first write); outputs listed in ``self.fused_acc`` are written / accumulated by the
        producing kernel itself and come back as the accumulator buffer."""
        env: Dict[int, Any] = dict(zip(self.inputs, inputs))
        if isinstance(inputs, list):
            inputs.clear()  # the environment is now the only owner of handed-over inputs
        for idx, ins in enumerate(self.instrs):
            kind = ins.kind
            if kind == 6:  # operator that writes straight into a gradient accumulator
                args = _materialize(ins.args, env, ctx)
                kwargs = _materialize(ins.kwargs, env, ctx)
                pos, dtype = ins.extra
                buf = acc_bufs[pos] if acc_bufs is not None else None
                env[ins.outs[0]] = ins.fn(*args, acc=(buf, dtype), **kwargs)
            elif kind == 0:  # captured operator
                args = ins.args if ins.static else _materialize(ins.args, env, ctx)
                kwargs = ins.kwargs if ins.static else _materialize(ins.kwargs, env, ctx)
                res = ins.fn(*args, **kwargs)
                if ins.slots is None:
                    env[ins.outs[0]] = res
                else:
                    for pos, slot in enumerate(ins.slots):
                        if slot is not None:
                            env[ins.outs[slot]] = res[pos]
            elif kind == 1:  # identity-like
                env[ins.outs[0]] = env[ins.args]
            elif kind == 2:  # copy
                env[ins.outs[0]] = env[ins.args].clone()
            elif kind == 3:  # dynamic slice at a host-provided offset
                dim, size, shards = ins.extra
                x = env[ins.args]
                piece = x.narrow(dim, scalars[0] // shards, size // shards)
                # rows of the leading dimension are one block of memory; a slice of an inner
                # dimension is not, and the captured operators (views) expect a dense operand
                env[ins.outs[0]] = piece if piece.is_contiguous() else piece.contiguous()
            elif kind == 4:  # all-reduce over mesh axes
                axes, scale, in_place = ins.extra
                y = ctx.all_reduce(env[ins.args], axes, ins.node_id, in_place=in_place)
                if scale != 1.0:
                    y = y.mul_(scale) if in_place else y * scale
                env[ins.outs[0]] = y
            elif kind == 5:  # local reshard
                src, dst = ins.extra
                env[ins.outs[0]] = ctx.spmd_reshard(env[ins.args], src, dst, ins.node_id)
            elif kind == 8:  # operator whose per-device form exchanges data with other devices of the task
                fn, axes = ins.extra
                args = _materialize(ins.args, env, ctx)
                res = fn(ctx, axes, ins.node_id, *args)
                if ins.slots is None:
                    env[ins.outs[0]] = res
                else:
                    for pos, slot in enumerate(ins.slots):
                        if slot is not None:
                            env[ins.outs[slot]] = res[pos]
            elif kind == 7:  # linear whose partial result is all-reduced: one fused kernel
                axes, scale, is_dgrad = ins.extra
                x, w = _materialize(ins.args, env, ctx)
                y = ctx.linear_all_reduce(x, w, axes, is_dgrad, ins.node_id)
                env[ins.outs[0]] = y if scale == 1.0 else y * scale
            elif kind == 9:  # reduce-scatter of a partial result
                axes, scale, dim, src, dst = ins.extra
                y = ctx.reduce_scatter(env[ins.args], axes, dim, src, dst, ins.node_id)
                env[ins.outs[0]] = y if scale == 1.0 else y.mul_(scale)
            elif kind == 10:  # linear whose partial result is reduce-scattered: one fused kernel
                axes, scale, is_dgrad, dim, src, dst = ins.extra
                x, w = _materialize(ins.args, env, ctx)
                y = ctx.linear_reduce_scatter(x, w, axes, is_dgrad, dim, src, dst, ins.node_id)
                env[ins.outs[0]] = y if scale == 1.0 else y.mul_(scale)
            elif kind == 11:  # all-gather of the row-sharded activation fused into the linear that reads it
                is_dgrad, axes, dim, src, dst, gathered_vid, x_vid, w_vid = ins.extra
                y, full = ctx.all_gather_linear(env[x_vid], env[w_vid], is_dgrad, axes, dim, src, dst, ins.node_id)
                env[gathered_vid] = full
                env[ins.outs[0]] = y
            # free values whose last use was this instruction (keeps peak memory low)
            dead = self._last_use.get(idx)
            if dead:
                for v in dead:
                    env.pop(v, None)
        return [env[v] for v in self.outputs]


def _local_shape(value: dict) -> List[int]:
    sh = value.get("sharding")
    return list(sh["shard_size"]) if sh else list(value["shape"])


def build_program(cap: Captured, plan: dict, template: dict, fast_ops: Optional[Dict[str, Callable]] = None,
                  acc_fusable: Optional[set] = None) -> TemplateProgram:
    g = cap.graph
    instrs: List[Instr] = []
    fast_variants: List[Tuple[Instr, Callable, str]] = []   # (instruction, plain operator, op name)
    single_device = template["num_devices"] == 1
    fx_by_name = getattr(cap, "_fx_by_name", None)
    if fx_by_name is None:
        fx_by_name = {n.name: n for n in cap.gm.graph.nodes}
        cap._fx_by_name = fx_by_name
    for nid in template["nodes"]:
        n = g.node(nid)
        op = n["op"]
        # nodes cloned by the compiler (recompute / replication) carry the name of their fx origin
        fxn = cap.fx_of_node.get(nid) or fx_by_name.get(n["attrs"].get("fx", ""))
        if fxn is not None and not op.startswith("mm."):
            # argument structure: fx nodes -> current IR inputs (passes may have rewired them)
            tensor_inputs = iter(n["inputs"])
            orig_inputs: Dict[fx.Node, int] = {}

            def conv(a):
                if isinstance(a, fx.Node):
                    key = a
                    if key not in orig_inputs:
                        vid = _ir_value_of(cap, a)
                        if vid is None:
                            raise NotImplementedError(f"non-tensor fx value {a} used by {fxn}")
                        orig_inputs[key] = vid
                    return _V(orig_inputs[key])
                if isinstance(a, torch.device):
                    return _Dev()
                if isinstance(a, (list, tuple)):
                    return type(a)(conv(e) for e in a) if isinstance(a, tuple) else [conv(e) for e in a]
                if isinstance(a, dict):
                    return {k: conv(v) for k, v in a.items()}
                return a

            args = tuple(conv(a) for a in fxn.args)
            kwargs = {k: conv(v) for k, v in fxn.kwargs.items()}
            # inputs may have been rewired by passes (e.g. reductions inserted): map old -> new positionally
            old_ids = _tensor_ids_in_order(args, kwargs)
            if len(old_ids) == len(n["inputs"]):
                remap = {o: nw for o, nw in zip(old_ids, n["inputs"]) if o != nw}
                if remap:
                    args = _remap(args, remap)
                    kwargs = _remap(kwargs, remap)
            # global -> local shapes in size arguments of sharded results
            if not single_device and op in _SIZE_ARG_OPS and n["outputs"]:
                outv = g.value(n["outputs"][0])
                gshape, lshape = list(outv["shape"]), _local_shape(outv)
                if gshape != lshape:
                    args = tuple(_fix_sizes(a, gshape, lshape) for a in args)
            fn = fxn.target
            if n["attrs"].get("zero_result") == "1":
                fn = _zeroed(fxn.target)
            if fast_ops and op in fast_ops:
                fn = fast_ops[op]
                fast_pending = (fxn.target, op)
            else:
                fast_pending = None
            val = fxn.meta.get("val")
            single = isinstance(val, torch.Tensor)
            slots = None
            if not single:
                slots, k = [], 0
                for e in val:
                    if isinstance(e, torch.Tensor):
                        slots.append(k)
                        k += 1
                    else:
                        slots.append(None)
            instrs.append(Instr(0, fn, args, kwargs, n["outputs"], None if single else slots, nid))
            shared = n["attrs"].get("shared_axes")
            if shared is not None and not single_device and json.loads(shared):
                from ..ops import moe as _moe  # noqa: F401  (registers its entries)
                from ..ops.mm_ops import CTX_OPS
                if op in CTX_OPS:
                    instrs[-1].kind = 8
                    instrs[-1].extra = (CTX_OPS[op][0], json.loads(shared))
                    instrs[-1].static = False
            if fast_pending is not None:
                fast_variants.append((instrs[-1],) + fast_pending)
            continue
        attrs = n["attrs"]
        if op in ("mm.accumulate", "mm.relayout") or op.startswith("mm.marker"):
            instrs.append(Instr(1, None, n["inputs"][0], None, n["outputs"], None, nid))
        elif op == "mm.copy":
            instrs.append(Instr(2, None, n["inputs"][0], None, n["outputs"], None, nid))
        elif op == "mm.dynamic_slice":
            dim, size = int(attrs["dim"]), int(attrs["size"])
            shards = 1
            sh = g.value(n["outputs"][0]).get("sharding")
            if sh and not single_device:
                for a in sh["dim_axes"][dim]:
                    shards *= sh["mesh_dims"][a]
            instrs.append(Instr(3, None, n["inputs"][0], None, n["outputs"], None, nid, (dim, size, shards)))
        elif op == "mm.all_reduce":
            axes = json.loads(attrs["axes"])
            instrs.append(Instr(4, None, n["inputs"][0], None, n["outputs"], None, nid,
                                (axes, float(attrs["scale"]), attrs.get("in_place") == "1")))
        elif op == "mm.spmd_reshard":
            from .. import _mm_C
            src = _mm_C.sharded_shape_from_json(attrs["from"])
            dst = _mm_C.sharded_shape_from_json(attrs["to"])
            instrs.append(Instr(5, None, n["inputs"][0], None, n["outputs"], None, nid, (src, dst)))
        elif op == "mm.reduce_scatter":
            from .. import _mm_C
            src = _mm_C.sharded_shape_from_json(attrs["from"])
            dst = _mm_C.sharded_shape_from_json(attrs["to"])
            instrs.append(Instr(9, None, n["inputs"][0], None, n["outputs"], None, nid,
                                (json.loads(attrs["axes"]), float(attrs["scale"]), int(attrs["dim"]), src, dst)))
        else:
            raise NotImplementedError(f"no lowering for compiler-generated op {op}")
    # identity-like instructions (layout markers, accumulate markers) only rename a value: readers
    # take the operand directly, so that the fusions below see producer and consumer side by side
    if not single_device:
        outputs_set = set(template["outputs"])
        rename: Dict[int, int] = {}
        kept: List[Instr] = []
        tail: List[Instr] = []
        for ins in instrs:
            if rename:
                if ins.kind in (0, 6):
                    ins.args = _remap(ins.args, rename)
                    ins.kwargs = _remap(ins.kwargs, rename)
                elif isinstance(ins.args, int) and ins.args in rename:
                    ins.args = rename[ins.args]
            if ins.kind == 1 and g.node(ins.node_id)["op"] != "mm.accumulate":
                rename[ins.outs[0]] = ins.args
                if ins.outs[0] in outputs_set:
                    tail.append(ins)        # still defines a task output: bound at the end of the program
                continue
            kept.append(ins)
        instrs = kept + tail
    # fuse "linear -> all-reduce of its partial result" into one GEMM+collective kernel
    if not single_device:
        readers: Dict[int, List[Instr]] = {}
        for ins in instrs:
            for v in _reads(ins):
                readers.setdefault(v, []).append(ins)
        outputs_set = set(template["outputs"])
        removed = set()
        for ins in instrs:
            if ins.kind != 0 or ins.slots is not None or not ins.outs:
                continue
            opname = g.node(ins.node_id)["op"]
            if opname not in ("mm_ops.linear.default", "mm_ops.linear_dgrad.default"):
                continue
            v = ins.outs[0]
            rd = readers.get(v, [])
            if len(rd) != 1 or rd[0].kind not in (4, 9) or v in outputs_set:
                continue
            ar = rd[0]
            is_dgrad = opname == "mm_ops.linear_dgrad.default"
            if ar.kind == 4:
                axes, scale, _ = ar.extra
                ins.kind = 7
                ins.extra = (axes, scale, is_dgrad)
            else:
                axes, scale, dim, src, dst = ar.extra
                # the scattered dimension must be one of the row dimensions of the product
                wv = g.value(g.node(ins.node_id)["inputs"][1])
                n_rows_dims = len(g.value(v)["shape"]) - ((len(wv["shape"]) - 1) if not is_dgrad else 1)
                if dim >= n_rows_dims:
                    continue
                ins.kind = 10
                ins.extra = (axes, scale, is_dgrad, dim, src, dst)
            ins.outs = ar.outs
            removed.add(id(ar))
        if removed:
            instrs = [i for i in instrs if id(i) not in removed]
        # fuse "all-gather of a row-sharded activation -> linear" into one kernel that also
        # returns the gathered activation (the backward pass needs it for the weight gradient)
        removed = set()
        position = {id(ins): k for k, ins in enumerate(instrs)}
        for ins in instrs:
            if ins.kind != 5:
                continue
            gattrs = g.node(ins.node_id)["attrs"]
            if "gather_dim" not in gattrs:
                continue
            gv = ins.outs[0]
            rd = readers.get(gv, [])
            live = sorted((r for r in rd if id(r) in position), key=lambda r: position[id(r)])
            def_pos = {v: position[id(i2)] for i2 in instrs for v in (i2.outs or ()) if id(i2) in position}
            first, ids = None, None
            task_inputs = set(template["inputs"])
            for k_r, r in enumerate(live):
                if r.kind != 0 or r.slots is not None:
                    continue
                if g.node(r.node_id)["op"] not in ("mm_ops.linear.default", "mm_ops.linear_dgrad.default"):
                    continue
                r_ids = _tensor_ids_in_order(r.args, r.kwargs)
                if len(r_ids) != 2 or r_ids[0] != gv or r_ids[1] == gv:
                    continue
                # a later reader can take the first reader's place when its other operand exists
                # from the start of the task (a weight)
                if k_r > 0 and r_ids[1] not in task_inputs and def_pos.get(r_ids[1], 1 << 30) > position[id(live[0])]:
                    continue
                first, ids = r, r_ids
                break
            if first is None:
                continue
            opname = g.node(first.node_id)["op"]
            if first is not live[0]:
                instrs.remove(first)
                instrs.insert(instrs.index(live[0]), first)
                position = {id(i2): k2 for k2, i2 in enumerate(instrs)}
            dim = int(gattrs["gather_dim"])
            if dim >= len(g.value(gv)["shape"]) - 1:
                continue                                  # only row dimensions of the activation
            src, dst = ins.extra
            first.kind = 11
            first.extra = (opname == "mm_ops.linear_dgrad.default", json.loads(gattrs["gather_axes"]), dim, src, dst,
                           gv, ins.args, ids[1])
            first.static = False
            removed.add(id(ins))
        if removed:
            instrs = [i for i in instrs if id(i) not in removed]
    # fuse "operator -> accumulate -> task output" into the operator's own epilogue
    fused_acc: Dict[int, bool] = {}
    if acc_fusable:
        out_pos = {v: k for k, v in enumerate(template["outputs"])}
        reads_count: Dict[int, int] = {}
        for ins in instrs:
            for v in _reads(ins):
                reads_count[v] = reads_count.get(v, 0) + 1
        by_out = {ins.outs[0]: ins for ins in instrs if ins.outs}
        for ins in instrs:
            if ins.kind != 1 or g.node(ins.node_id)["op"] != "mm.accumulate":
                continue
            if ins.outs[0] not in out_pos:
                continue
            prod = by_out.get(ins.args)
            if prod is None or prod.kind != 0 or reads_count.get(ins.args, 0) != 1 or ins.args in out_pos:
                continue
            if g.node(prod.node_id)["op"] not in acc_fusable or prod.slots is not None:
                continue
            pos = out_pos[ins.outs[0]]
            acc_dtype = DTYPE_FROM_NAME[g.value(ins.outs[0])["dtype"]]
            prod.kind = 6
            prod.extra = (pos, acc_dtype)
            fused_acc[pos] = True
    # liveness inside the program
    last: Dict[int, int] = {}
    keep = set(template["outputs"])
    for idx, ins in enumerate(instrs):
        for v in _reads(ins):
            last[v] = idx
    # A fast variant that overwrites one of its operands is only valid when nothing reads that
    # operand afterwards (passes may have moved a reader behind it): otherwise run the plain one.
    if fast_variants:
        from ..ops.mm_ops import INPLACE_OPERANDS
        # an input that another task reads as well (the two halves of a split backward task share
        # the incoming boundary gradient) must survive this task unchanged
        mine = set(template["inputs"])
        shared_inputs = {v for t in plan["templates"] if t is not template and t["name"] != template["name"]
                         for v in t["inputs"] if v in mine}
        index_of = {id(ins): idx for idx, ins in enumerate(instrs)}
        for ins_obj, plain, opname in fast_variants:
            idx = index_of.get(id(ins_obj))
            clobbered = INPLACE_OPERANDS.get(opname)
            if idx is None or not clobbered:
                continue
            ids = _tensor_ids_in_order(ins_obj.args, ins_obj.kwargs)
            for pos in clobbered:
                if pos < len(ids) and (last.get(ids[pos], -1) > idx or ids[pos] in keep or ids[pos] in shared_inputs):
                    ins_obj.fn = plain
                    break
    last_use: Dict[int, List[int]] = {}
    for v, idx in last.items():
        if v not in keep:
            last_use.setdefault(idx, []).append(v)
    prog = TemplateProgram(template, instrs, list(template["inputs"]), list(template["outputs"]), last_use)
    prog.fused_acc = fused_acc
    return prog


def _zeroed(target: Callable) -> Callable:
    """``target`` with its tensor result replaced by zeros of the same shape and type."""
    def run(*args, **kwargs):
        return torch.zeros_like(target(*args, **kwargs))
    return run


def _ir_value_of(cap: Captured, node: fx.Node) -> Optional[int]:
    return cap.value_of_fx.get((node, None))


def _tensor_ids_in_order(args, kwargs) -> List[int]:
    out: List[int] = []

    def walk(s):
        if isinstance(s, _V):
            out.append(s.vid)
        elif isinstance(s, (tuple, list)):
            for e in s:
                walk(e)
        elif isinstance(s, dict):
            for e in s.values():
                walk(e)

    walk(args)
    walk(kwargs)
    return out


def _remap(spec, remap):
    if isinstance(spec, _V):
        return _V(remap.get(spec.vid, spec.vid))
    if isinstance(spec, tuple):
        return tuple(_remap(s, remap) for s in spec)
    if isinstance(spec, list):
        return [_remap(s, remap) for s in spec]
    if isinstance(spec, dict):
        return {k: _remap(v, remap) for k, v in spec.items()}
    return spec


def _fix_sizes(arg, gshape, lshape):
    if isinstance(arg, (list, tuple)) and len(arg) == len(gshape) and all(isinstance(e, int) for e in arg):
        if all(a == b or a == -1 for a, b in zip(arg, gshape)):
            fixed = [l if a != -1 else -1 for a, l in zip(arg, lshape)]
            return type(arg)(fixed) if isinstance(arg, tuple) else fixed
    return arg


def _reads(ins: Instr) -> List[int]:
    if ins.kind == 11:      # reads the row shard (not the gathered value its operator names) and the weight
        return [ins.extra[6], ins.extra[7]]
    if ins.kind in (0, 6, 7, 10):
        return _tensor_ids_in_order(ins.args, ins.kwargs)
    return [ins.args]
