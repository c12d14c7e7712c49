"""The compiled step: per-step dispatch loop over the plan.

``Executable.__call__`` mirrors ``MultiMeshPjRtExecutable::Execute``
(``src/pjrt_client/mm_pjrt_executable.cc:271-708``): open a window, bind
parameter stores (reusing the tiles of sharded inputs, or slicing global
tensors into tiles), then walk the linear operation list and *submit* every
task and reshard for each local device to the native task-graph runtime, which
orders them by their store accesses; results are handed back as
:class:`ShardedTensor` objects whose tiles become valid when the step's tasks
have run (reading one blocks, nothing else does).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import threading

import torch
from torch.utils import _pytree as pytree

from .. import state
from ..compiler.capture import Captured, DTYPE_FROM_NAME
from ..compiler.lower import TemplateProgram, build_program
from ..ops import kernels as K
from .collectives import DeviceCtx, Rendezvous, Topology, tile_box


import weakref

live_executables: "weakref.WeakSet" = weakref.WeakSet()


class StepFailed(RuntimeError):
    """A task of the step reported an error (status code from the runtime)."""


class ShardedTensor:
    """A logical array stored as one tile per owning device.

    ``sharding`` is the descriptor dict produced by the compiler (dtype, global
    sizes, mesh axes per dimension, mesh shape, device range). Only tiles of
    devices local to this process are held."""

    def __init__(self, sharding: dict, tiles: Dict[int, torch.Tensor], topology: Topology, waiter=None, checker=None):
        self.sharding = sharding
        self._tiles = tiles
        self.topology = topology
        self._waiter = waiter
        self._checker = checker     # checker(block): raises if a kernel of the producing step failed

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(self.sharding["sizes"])

    @property
    def dtype(self) -> torch.dtype:
        return DTYPE_FROM_NAME[self.sharding["dtype"]]

    @property
    def devices(self) -> range:
        s = self.sharding["device_start"]
        return range(s, s + self.sharding["num_devices"])

    def wait(self) -> "ShardedTensor":
        if self._waiter is not None:
            w, self._waiter = self._waiter, None
            w()
        return self

    def local_tiles(self) -> Dict[int, torch.Tensor]:
        self.wait()
        return dict(self._tiles)

    def tile(self, device: int) -> torch.Tensor:
        self.wait()
        return self._tiles[device]

    def has_local_tile(self) -> bool:
        return any(self.topology.is_local(d) for d in self.devices)

    def full_tensor(self) -> torch.Tensor:
        """Assembles the global value (on the first local device, or CPU)."""
        self.wait()
        if self._checker is not None:
            self._checker(True)     # the value is about to be read: make sure no kernel reported a failure
        topo = self.topology
        sizes = self.sharding["sizes"]
        start = self.sharding["device_start"]
        if topo.kind != "dist":
            first = self._tiles[start]
            out = torch.empty(sizes, dtype=first.dtype, device=first.device)
            for d in self.devices:
                lo, hi = tile_box(self.sharding, d - start)
                out[tuple(slice(a, b) for a, b in zip(lo, hi))] = self._tiles[d].to(first.device)
            return out
        import torch.distributed as dist
        dev = topo.torch_device(topo.rank)
        replicated = all(len(a) == 0 for a in self.sharding["dim_axes"])
        if replicated and self.sharding["num_devices"] == topo.num_devices:
            return self._tiles[topo.rank]      # every rank already holds the whole value
        out = torch.empty(sizes, dtype=self.dtype, device=dev)
        for d in self.devices:
            lo, hi = tile_box(self.sharding, d - start)
            shape = [b - a for a, b in zip(lo, hi)]
            buf = self._tiles[d].contiguous() if d == topo.rank else torch.empty(shape, dtype=self.dtype, device=dev)
            dist.broadcast(buf, src=d)
            out[tuple(slice(a, b) for a, b in zip(lo, hi))] = buf
        return out

    def item(self):
        return self.full_tensor().item()

    def __repr__(self):
        return f"ShardedTensor({self.sharding['key']})"


def shard_tensor(t: torch.Tensor, sharding: dict, topology: Topology, private: bool = False) -> ShardedTensor:
    """Slices a global tensor into the tiles of ``sharding`` (local devices only). Tiles are
    contiguous; with ``private`` they never share storage with ``t`` (needed for arguments
    that were not donated, because compiled tasks may update dead inputs in place)."""
    tiles: Dict[int, torch.Tensor] = {}
    start = sharding["device_start"]
    seen_shared = False
    for o in range(sharding["num_devices"]):
        d = start + o
        if not topology.is_local(d):
            continue
        lo, hi = tile_box(sharding, o)
        piece = t[tuple(slice(a, b) for a, b in zip(lo, hi))]
        tile = piece.to(topology.torch_device(d)).contiguous()
        shares = tile.untyped_storage().data_ptr() == t.untyped_storage().data_ptr()
        if shares and (private or seen_shared):
            tile = tile.clone()   # virtual devices of one process must not share a buffer either
        seen_shared = seen_shared or shares
        tiles[d] = tile
    return ShardedTensor(sharding, tiles, topology)


class Executable:
    def __init__(self, cap: Captured, plan: dict, topology: Topology, *, context=None, name: str = "step",
                 fast_ops: Optional[Dict[str, Any]] = None, acc_fusable: Optional[set] = None):
        from .. import _mm_C
        if fast_ops is None:
            try:
                from ..ops.mm_ops import ACC_FUSABLE, FAST_OPS
                fast_ops, acc_fusable = FAST_OPS, ACC_FUSABLE
            except Exception:  # pragma: no cover
                fast_ops = None
        self.cap = cap
        self.plan = plan
        self.topology = topology
        self.name = name
        self.programs: Dict[int, TemplateProgram] = {}
        # a process builds the programs of the templates it will run: those compiled for its devices
        # and those that some operation of the plan places there (a task that moves between
        # sub-meshes per microbatch runs one template on several device ranges)
        runs_here = {op["template"] for op in plan["ops"] if op["kind"] == "task" and
                     any(topology.is_local(d) for d in range(op["device_start"], op["device_start"] + op["num_devices"]))}
        for t in plan["templates"]:
            local = t["id"] in runs_here or any(topology.is_local(d) for d in self._template_devices(t))
            if local or topology.kind != "dist":
                self.programs[t["id"]] = build_program(cap, plan, t, fast_ops, acc_fusable)
        # A process that drives exactly one CUDA device gets the context that owns the device's
        # streams: tasks on the caller's compute stream, reshards and once-per-step collectives on
        # a communication stream, ordered by CUDA events wherever the dependence analysis finds a
        # pair of conflicting accesses on different streams (MM_CUDA_CONTEXT=0: everything on one
        # stream through the host-side context).
        self._streams: Dict[int, Any] = {}
        self._cuda_ctx = False
        if context is None:
            import os
            inline = len(topology.local_devices) == 1
            dev0 = topology.torch_device(topology.local_devices[0])
            if inline and dev0.type == "cuda" and os.environ.get("MM_CUDA_CONTEXT", "1") != "0":
                d0 = topology.local_devices[0]
                ordinal = dev0.index if dev0.index is not None else torch.cuda.current_device()
                with torch.cuda.device(dev0):
                    compute = torch.cuda.current_stream(dev0).cuda_stream
                context = _mm_C.CudaContext([d0], [ordinal], [compute])
                context.set_task_ranges(bool(state.knobs["task_ranges"]))
                for kind in (1, 2):
                    self._streams[kind] = torch.cuda.ExternalStream(context.stream_handle(d0, kind), device=dev0)
                self._cuda_ctx = True
            else:
                context = _mm_C.ThreadedContext(topology.local_devices, inline, False)
        self.context = context
        import os as _os
        self._overlap_reduce = _os.environ.get("MM_OVERLAP_REDUCE", "1") != "0"
        self._compute_stream = None
        if self._cuda_ctx:
            dev0 = topology.torch_device(topology.local_devices[0])
            self._compute_stream = torch.cuda.current_stream(dev0)
        self.rendezvous = Rendezvous()
        self.dev_ctx = {d: DeviceCtx(topology, d, self.rendezvous) for d in topology.local_devices}
        topology.prepare_groups(sorted({(t["device_start"], tuple(t["mesh_dims"])) for t in plan["templates"]}))
        # physical buffers: stores sharing a scheduling name and layout share one id
        self.buffer_of: Dict[int, int] = {}
        names: Dict[str, int] = {}
        for st in plan["stores"]:
            root = st
            while root["alias_of"] >= 0:
                root = plan["stores"][root["alias_of"]]
            key = root["name"] + "@" + root["shape"]["key"]
            self.buffer_of[st["id"]] = names.setdefault(key, len(names))
        # stores that share a physical buffer share one tile table: writing a store drops the
        # tensor of the store that used the buffer before (the compiler's liveness plan)
        self._buffer_tiles: Dict[int, Dict[int, torch.Tensor]] = {}
        self.tiles: Dict[int, Dict[int, torch.Tensor]] = {
            st["id"]: self._buffer_tiles.setdefault(self.buffer_of[st["id"]], {}) for st in plan["stores"]}
        self._step = 0
        self._created = False
        self._reshard_plans: Dict[Tuple[int, int], dict] = {}
        # per-step invariants of the dispatch loop, built at first submission and reused
        self._task_entries: Dict[Tuple[int, int], tuple] = {}
        self._in_use: Dict[int, int] = {}          # lifetime checking: storages of tiles handed to running tasks
        self._in_use_lock = threading.Lock()
        self._reshard_entries: Dict[int, list] = {}
        self._cur_step = 0
        self._cur_roots: Dict[int, Dict[int, torch.Tensor]] = {}
        self._setup_fused_tp()
        # one-process-per-GPU jobs: side stream for stage-boundary messages, and the events
        # that mark the arrival of a received tile, keyed by (buffer, device)
        self._comm: Dict[int, Any] = {}
        self._arrival: Dict[Tuple[int, int], Any] = {}
        self.launches = 0
        self._inline = len(topology.local_devices) == 1
        # kernel status words of the local CUDA devices, read without stalling the streams
        self._probes = {d: K.StatusProbe(topology.torch_device(d)) for d in topology.local_devices
                        if topology.torch_device(d).type == "cuda"}
        self.donated = set(getattr(cap, "donated_inputs", ()))
        # Temporaries handed over to their last reader (task op k), which frees each one right after
        # its last use. Readers of one tile are not ordered among themselves by the dependence
        # analysis, so this is only safe when they cannot overtake one another: every reader is a
        # task of a strict-order chain (on one device those run in plan order) and no reshard -
        # which runs on its own thread - reads the store at all.
        last_read: Dict[int, int] = {}
        unsafe: set = set()
        for k, op in enumerate(plan["ops"]):
            if op["kind"] == "task":
                for sid in op["inputs"]:
                    last_read[sid] = k
                    if not op["strict_ordering"]:
                        unsafe.add(sid)
                for sid, m in zip(op["outputs"], op["accumulate"]):
                    if m:
                        unsafe.add(sid)              # accumulators are read-modify-written: never hand over
            elif op["kind"] == "reshard":
                unsafe.add(op["src_store"])
        self._dying_inputs: Dict[int, set] = {}
        for sid, k in last_read.items():
            st = plan["stores"][sid]
            if sid not in unsafe and st["kind"] == "TEMP" and st["alias_of"] < 0:
                self._dying_inputs.setdefault(k, set()).add(sid)
        self._build_native_programs()
        # Debug aid for the compiler's buffer plan (MM_CHECK_LIFETIMES=1): stores that share a
        # physical buffer must never be alive at the same time. With the knob on, every tile
        # remembers which store wrote it last; a task or reshard that reads a store whose buffer
        # has meanwhile been handed to another store fails the step with both names, and the
        # tile that loses its buffer is filled with NaN first, so that a kernel still holding the
        # old address produces visibly wrong numbers instead of plausible ones.
        import os as _os2
        self._lifetimes = _os2.environ.get("MM_CHECK_LIFETIMES", "0") == "1"
        self._owner: Dict[Tuple[int, int], int] = {}
        self._alias_root: Dict[int, int] = {}
        for st in plan["stores"]:
            root = st
            while root["alias_of"] >= 0:
                root = plan["stores"][root["alias_of"]]
            self._alias_root[st["id"]] = root["id"]
        live_executables.add(self)

    def _took_buffer(self, sid: int, d: int, old: Optional[torch.Tensor], new: torch.Tensor) -> None:
        """Store ``sid`` has just been written on device ``d`` (lifetime checking only)."""
        key = (self.buffer_of[sid], d)
        me = self._alias_root[sid]
        prev = self._owner.get(key)
        if prev is not None and prev != me and old is not None and old is not new and old.is_floating_point() \
                and old.untyped_storage().data_ptr() != new.untyped_storage().data_ptr() and not self._in_arena(old) \
                and not self._storage_shared(old):
            # (tiles inside the peer-mapped arena are left alone: another GPU may still be pulling them;
            # so is memory that another store's tile is a view of - two results of one task, a detached
            # copy - since that store may be read long after this buffer's name was handed on)
            old.fill_(float("nan"))
        self._owner[key] = me

    def _storage_shared(self, t: torch.Tensor) -> bool:
        ptr = t.untyped_storage().data_ptr()
        with self._in_use_lock:
            if ptr in self._in_use:          # a running task of another thread still reads a view of it
                return True
        for tiles in self.tiles.values():
            for other in tiles.values():
                if other is not t and isinstance(other, torch.Tensor) and other.untyped_storage().data_ptr() == ptr:
                    return True
        return False

    def _in_arena(self, t: torch.Tensor) -> bool:
        pr = getattr(self, "_peer_reshard", None)
        if pr is None or not t.is_cuda:
            return False
        a = pr.arena
        return a.base <= t.data_ptr() < a.base + a.nbytes

    def _check_owner(self, sid: int, d: int, reader: str) -> None:
        key = (self.buffer_of[sid], d)
        owner = self._owner.get(key)
        if owner is not None and owner != self._alias_root[sid]:
            a, b = self.plan["stores"][sid], self.plan["stores"][owner]
            raise RuntimeError(f"{reader} reads store {sid} ({a['name']}, {a['shape']['key']}) on device {d}, but its buffer "
                               f"was handed to store {owner} ({b['name']}) in the meantime: the buffer plan lets two live "
                               "stores share a buffer")

    def _build_native_programs(self) -> None:
        """Kernel programs for the templates that are nothing but calls into the kernel library
        (see :mod:`multimesh_jax_b200.compiler.native`): their task bodies then run as one call into
        the C++ launcher over memory planned ahead of time - task outputs carved from one block
        per launch, intermediates at fixed offsets of the runtime context's scratch tile.
        Templates with collectives, and anything on CPU devices, keep the interpreted program.
        MM_NATIVE_TASKS=0 switches the native path off."""
        import os
        self._native: Dict[Tuple[int, bool], Any] = {}
        self._native_why: Dict[int, str] = {}
        self._scratch_base: Dict[int, int] = {}
        self._native_off: set = set()
        self.native_launches = 0
        if not self._cuda_ctx or os.environ.get("MM_NATIVE_TASKS", "1") == "0":
            return
        from ..compiler.native import NativeUnsupported, build_native
        patterns: Dict[int, set] = {}
        for op in self.plan["ops"]:
            if op["kind"] == "task" and op["template"] in self.programs:
                modes = tuple(op["accumulate"])
                if any(m == 1 for m in modes) and any(m == 2 for m in modes):
                    self._native_why[op["template"]] = "mixed first-write / accumulate outputs"
                    patterns[op["template"]] = None
                    continue
                if patterns.get(op["template"], set()) is not None:
                    patterns.setdefault(op["template"], set()).add((tuple(1 if m else 0 for m in modes), any(m == 2 for m in modes)))
        # Outputs that a pull-kernel reshard reads are written straight into the reshard's
        # peer-mapped tile (every launch of the template must agree on it), and inputs that a
        # reshard reads are never overwritten in place: the pull runs on another GPU, outside
        # this device's ordering.
        pr = self._peer_reshard
        reshard_src = {op["src_store"] for op in self.plan["ops"] if op["kind"] == "reshard"}
        readers: Dict[int, set] = {}
        for op in self.plan["ops"]:
            if op["kind"] == "reshard":
                readers.setdefault(op["src_store"], set()).add((self.buffer_of[op["src_store"]], self.buffer_of[op["dst_store"]]))
        # store -> the one reshard slot that reads it (stores read by several reshards, or by one
        # that goes through NCCL, keep tiles of their own and are copied)
        self._direct_key: Dict[int, tuple] = {}
        if pr is not None and os.environ.get("MM_RESHARD_DIRECT", "1") != "0":
            for sid, keys in readers.items():
                if len(keys) == 1 and pr.slots.get(next(iter(keys))) is not None:
                    self._direct_key[sid] = next(iter(keys))
        ext: Dict[int, set] = {}
        protect: Dict[int, set] = {}
        for op in self.plan["ops"]:
            if op["kind"] != "task":
                continue
            direct = {k for k, (sid, m) in enumerate(zip(op["outputs"], op["accumulate"]))
                      if m == 0 and sid in self._direct_key}
            tid = op["template"]
            ext[tid] = direct if tid not in ext else ext[tid] & direct
            protect.setdefault(tid, set()).update(i for i, sid in enumerate(op["inputs"]) if sid in reshard_src)
        self._native_ext = {tid: sorted(v) for tid, v in ext.items()}
        scratch = 0
        for t in self.plan["templates"]:
            pats = patterns.get(t["id"])
            if not pats:
                continue
            built = {}
            try:
                for classes, have_acc in pats:
                    built[(t["id"], have_acc)] = build_native(self.cap, self.plan, t, self.programs[t["id"]], classes, have_acc,
                                                              self._native_ext.get(t["id"], ()),
                                                              sorted(protect.get(t["id"], ())))
            except NativeUnsupported as e:
                self._native_why[t["id"]] = str(e)
                continue
            self._native.update(built)
            scratch = max([scratch] + [n.scratch_bytes for n in built.values()])
        self.native_scratch_bytes = scratch
        if self._native:
            for d in self.topology.local_devices:
                base = self.context.reserve_scratch(d, max(scratch, 1 << 20))
                if not base:
                    raise MemoryError(f"cannot reserve {scratch} bytes of task scratch on device {d}")
                self._scratch_base[d] = base

    def native_report(self) -> Dict[str, str]:
        """Per template: ``native (<n> kernel calls)`` or why it keeps the interpreted program."""
        out = {}
        for t in self.plan["templates"]:
            progs = [n for (tid, _), n in self._native.items() if tid == t["id"]]
            if progs and not any(tid == t["id"] for tid, _ in self._native_off):
                out[t["name"]] = f"native ({max(n.num_calls for n in progs)} kernel calls)"
            else:
                out[t["name"]] = "interpreted: " + self._native_why.get(t["id"], "not on a CUDA context")
        return out

    def _setup_fused_tp(self) -> None:
        """One-process-per-GPU CUDA jobs get a peer-mapped (IPC) arena, created here,
        collectively, so that no rank meets the handle exchange in the middle of a step. It
        carries (1) the receive buffers of the fused GEMM+all-reduce kernel when the plan
        contains all-reduces of partial GEMM results (MM_FUSED_TP=0: NCCL reduces them), and
        (2) the staging tiles and flags of cross-submesh reshards, which the destination
        pulls straight from peer HBM (MM_P2P_RESHARD=0: NCCL point-to-point messages)."""
        import os
        topo = self.topology
        self._fused_tp = None
        self._peer_reshard = None
        if topo.kind != "dist" or topo.torch_device(topo.rank).type != "cuda":
            return
        g = self.cap.graph
        want_tp = os.environ.get("MM_FUSED_TP", "1") != "0" and any(
            g.node(n)["op"] in ("mm.all_reduce", "mm.reduce_scatter") or "gather_dim" in g.node(n)["attrs"]
            for t in self.plan["templates"] for n in t["nodes"])
        want_rs = os.environ.get("MM_P2P_RESHARD", "1") != "0" and any(
            op["kind"] == "reshard" for op in self.plan["ops"])
        moe_nodes = [g.node(n) for t in self.plan["templates"] for n in t["nodes"]
                     if g.node(n)["op"].startswith("mm_ops.moe_ffn.") and g.node(n)["attrs"].get("shared_axes", "[]") != "[]"]
        want_moe = os.environ.get("MM_P2P_MOE", "1") != "0" and bool(moe_nodes)
        want_comm = os.environ.get("MM_P2P_COLLECTIVES", "1") != "0" and any(
            g.node(n)["op"] in ("mm.all_reduce", "mm.reduce_scatter", "mm.spmd_reshard")
            for t in self.plan["templates"] for n in t["nodes"])
        if not (want_tp or want_rs or want_moe or want_comm):
            return
        from ..parallel import symm
        from ..parallel.reshard import PeerReshard
        from .collectives import FusedTP
        nbytes = 1 << 20
        if want_tp:
            nbytes += int(os.environ.get("MM_SYMM_ARENA_MB", "1024")) << 20
        if want_rs:
            nbytes += PeerReshard.required_bytes(self.plan, self.buffer_of) + (1 << 20)
        if want_comm:
            # staging pairs of the in-task collectives: one pair per power-of-two size class and per
            # stream kind (once-per-step reductions run on the communication stream with tiles of their own)
            sizes = set()
            for t in self.plan["templates"]:
                kind = 1 if (self._cuda_ctx and self._overlap_reduce and t["name"].endswith("_reduce")) else 0
                for n in t["nodes"]:
                    nd = g.node(n)
                    if nd["op"] in ("mm.all_reduce", "mm.reduce_scatter", "mm.spmd_reshard"):
                        v = g.value(nd["inputs"][0])
                        nb = DTYPE_FROM_NAME[v["dtype"]].itemsize
                        for s_ in (v["sharding"]["shard_size"] if v["sharding"] else v["shape"]):
                            nb *= s_
                        if nb >= (256 << 10):
                            sizes.add((kind, 1 << max(20, (nb - 1).bit_length())))
            nbytes += 2 * sum(sz for _, sz in sizes) + (4 << 20)
        if want_moe:
            from ..parallel.ep import PeerMoE, PeerMoERegistry
            worst = 0
            for nd in moe_nodes:
                xv, wv = g.value(nd["inputs"][0]), g.value(nd["inputs"][2])
                tokens = 1
                for s_ in (xv["sharding"]["shard_size"] if xv["sharding"] else xv["shape"])[:-1]:
                    tokens *= s_
                worst = max(worst, PeerMoE.required_bytes(tokens, xv["shape"][-1], wv["shape"][0]))
            nbytes += worst
        arena = symm.SymmetricArena(nbytes, topo.torch_device(topo.rank))
        self._arena = arena
        if want_rs:
            self._peer_reshard = PeerReshard(arena, topo, self.plan, self.buffer_of, self._reshard_plan)
        if want_tp:
            self._fused_tp = FusedTP(arena)
            for ctx in self.dev_ctx.values():
                ctx.fused_tp = self._fused_tp
        if want_comm:
            from ..parallel.peer_comm import PeerCommRegistry
            self._peer_comm = PeerCommRegistry(arena)
            for ctx in self.dev_ctx.values():
                ctx.peer_comm = self._peer_comm
        if want_moe:
            self._peer_moe = PeerMoERegistry(arena)
            for ctx in self.dev_ctx.values():
                ctx.peer_moe = self._peer_moe

    def _comm_stream(self, d: int):
        """Side stream of device ``d`` for point-to-point messages (``None`` unless this is a
        one-process-per-GPU CUDA job; MM_COMM_STREAM=0 keeps messages on the compute stream)."""
        import os
        topo = self.topology
        if self._cuda_ctx:
            return None       # the runtime context owns the communication stream and orders the readers
        if topo.kind != "dist" or topo.torch_device(d).type != "cuda" or os.environ.get("MM_COMM_STREAM", "1") == "0":
            return None
        if d not in self._comm:
            from ..parallel.reshard import CommStream
            self._comm[d] = CommStream(topo.torch_device(d))
        return self._comm[d]

    @staticmethod
    def _template_devices(t: dict) -> range:
        return range(t["device_start"], t["device_start"] + t["num_devices"])

    # ------------------------------------------------------------------ inputs
    def input_shardings(self) -> List[Optional[dict]]:
        out = []
        for sid in self.plan["param_stores"]:
            out.append(self.plan["stores"][sid]["shape"] if sid >= 0 else None)
        return out

    def output_shardings(self) -> List[dict]:
        return [self.plan["stores"][sid]["shape"] for sid in self.plan["root_stores"]]

    def shard_argument(self, argnum: int, value: Any) -> Any:
        """Lays out argument ``argnum`` (a pytree of global tensors) as the
        compiled step expects it."""
        cap = self.cap
        example = pytree.tree_unflatten(list(range(len(cap.input_is_tensor))), cap.in_spec)
        positions = pytree.tree_leaves(example[argnum])
        tensor_index = {}
        k = 0
        for i, ok in enumerate(cap.input_is_tensor):
            if ok:
                tensor_index[i] = k
                k += 1
        leaves, spec = pytree.tree_flatten(value)
        out = []
        for pos, leaf in zip(positions, leaves):
            if pos in tensor_index and isinstance(leaf, torch.Tensor):
                sid = self.plan["param_stores"][tensor_index[pos]]
                out.append(shard_tensor(leaf, self.plan["stores"][sid]["shape"], self.topology) if sid >= 0 else leaf)
            else:
                out.append(leaf)
        return pytree.tree_unflatten(out, spec)

    # ------------------------------------------------------------------ run
    def __call__(self, *args):
        cap, plan, ctx, topo = self.cap, self.plan, self.context, self.topology
        flat, _ = pytree.tree_flatten(tuple(args))
        tensors = [a for a in flat if isinstance(a, (torch.Tensor, ShardedTensor))]
        if len(tensors) != cap.num_inputs:
            raise ValueError(f"expected {cap.num_inputs} tensor arguments, got {len(tensors)}")
        step = self._step
        self._step += 1
        if not self._inline:
            # parameter tiles are rebound below: the previous step must not be reading them any more
            status, msg = ctx.wait_all()
            if int(status) != 0:
                ctx.reset_error()
                raise StepFailed(f"{self.name}: {status.name}: {msg}")
            for probe in self._probes.values():
                with torch.cuda.device(probe.device):
                    probe.record()
        self._check_kernel_status(block=False)
        ctx.open_window()
        ctx.start_timer(self.name)
        ctx.mark_profile(f"start {self.name}")
        if not self._created:
            for st in plan["stores"]:
                nbytes = 1
                for s in st["shape"]["shard_size"]:
                    nbytes *= s
                nbytes *= DTYPE_FROM_NAME[st["shape"]["dtype"]].itemsize
                for d in range(st["shape"]["device_start"], st["shape"]["device_start"] + st["shape"]["num_devices"]):
                    if topo.is_local(d):
                        ctx.create_store(self.buffer_of[st["id"]], d, nbytes, False)
            self._created = True
        # parameter stores
        for i, sid in enumerate(plan["param_stores"]):
            if sid < 0:
                continue
            want = plan["stores"][sid]["shape"]
            a = tensors[i]
            if isinstance(a, ShardedTensor):
                if a.sharding["key"] != want["key"]:
                    a = shard_tensor(a.full_tensor(), want, topo)
                new_tiles = a.local_tiles()
            else:
                new_tiles = shard_tensor(a, want, topo, private=i not in self.donated).local_tiles()
            self.tiles[sid].clear()
            self.tiles[sid].update(new_tiles)
            if self._lifetimes:
                for d_ in new_tiles:
                    self._owner[(self.buffer_of[sid], d_)] = self._alias_root[sid]
        root_tiles: Dict[int, Dict[int, torch.Tensor]] = {sid: {} for sid in plan["root_stores"]}
        # the task bodies are built once per (operation, device) and kept; what changes from step to
        # step reaches them through these two fields (the previous step's bodies have all run: the
        # wait above, or inline submission)
        self._cur_step, self._cur_roots = step, root_tiles
        # dispatch loop
        for k, op in enumerate(plan["ops"]):
            kind = op["kind"]
            if kind == "task":
                for d in range(op["device_start"], op["device_start"] + op["num_devices"]):
                    if topo.is_local(d):
                        self._submit_task(k, op, d, step, root_tiles)
            elif kind == "reshard":
                self._submit_reshard(k, op, step, root_tiles)
        if self._comm:
            # bodies ran inline: every message of the step is queued; results handed to the
            # caller must be ordered behind them on the compute stream
            for d, comm in self._comm.items():
                with torch.cuda.device(comm.device):
                    comm.drain()
            self._arrival.clear()
        ctx.stop_timer(self.name)
        ctx.close_window()
        ctx.mark_profile(f"finish {self.name}")
        if self._probes and self._inline:
            for d, probe in self._probes.items():
                probe.record()      # bodies ran inline: the step's kernels are all queued
        # results
        waited = {"done": False}

        def waiter():
            if waited["done"]:
                return
            waited["done"] = True
            status, msg = ctx.wait_all()
            if int(status) != 0:
                ctx.reset_error()
                raise StepFailed(f"{self.name}: {status.name}: {msg}")
            self._check_kernel_status(block=False)

        outs: List[Any] = []
        it = iter(plan["root_stores"])
        n_out = len(cap.output_values) + len(cap.output_constants)
        for pos in range(n_out):
            if pos in cap.output_constants:
                outs.append(cap.output_constants[pos])
                continue
            sid = next(it)
            outs.append(ShardedTensor(plan["stores"][sid]["shape"], root_tiles[sid], topo, waiter,
                                      self._check_kernel_status if self._probes else None))
        return pytree.tree_unflatten(outs, cap.out_spec)

    # ------------------------------------------------------------------ tasks
    def _submit_task(self, k: int, op: dict, d: int, step: int, root_tiles):
        entry = self._task_entries.get((k, d))
        if entry is None:
            entry = self._task_entries[(k, d)] = self._make_task_entry(k, op, d)
        reads, writes, body, kind = entry
        self.launches += 1
        if self._cuda_ctx:
            self.context.create_execute_task(d, reads, writes, body, op["name"], op["strict_ordering"], op["priority"], step,
                                             kind)
        else:
            self.context.create_execute_task(d, reads, writes, body, op["name"], op["strict_ordering"], op["priority"], step)

    def _make_task_entry(self, k: int, op: dict, d: int):
        """Read / write tile lists, stream kind and body of operation ``k`` on device ``d``: everything
        about a task launch that does not change between steps, built at its first submission."""
        prog = self.programs[op["template"]]
        tiles = self.tiles
        dctx = self.dev_ctx[d]
        buf = self.buffer_of
        reads = [(buf[s], d) for s in op["inputs"]]
        writes = [(buf[s], d) for s in op["outputs"]]
        reads += [(buf[s], d) for s, m in zip(op["outputs"], op["accumulate"]) if m == 2]
        scalars = op["scalars"]
        in_ids, out_ids, modes = op["inputs"], op["outputs"], op["accumulate"]
        dev_start, mesh_dims = op["device_start"], prog.mesh_dims
        fused = prog.fused_acc
        dying = self._dying_inputs.get(k, ())
        acc_dtypes = [DTYPE_FROM_NAME[self.plan["stores"][s]["shape"]["dtype"]] for s in out_ids]
        stores = self.plan["stores"]
        in_shapes = [tuple(stores[s]["shape"]["shard_size"]) for s in in_ids]
        arrival = self._arrival
        in_keys = [(buf[s], d) for s in in_ids] + [(buf[s], d) for s, m in zip(out_ids, modes) if m == 2]

        name = op["name"]
        # once-per-step reductions that are tasks of their own run on the communication stream:
        # the reduction of one gradient overlaps the optimizer update of the previous ones
        kind = 0
        if self._cuda_ctx and name.endswith("_reduce") and self._overlap_reduce:
            kind = 1
        side = self._streams.get(kind)

        def body():
            if state.knobs["task_ranges"]:
                # one named range per task launch: visible to torch.profiler and, through NVTX, to
                # external timeline tools
                nvtx = dctx.torch_device.type == "cuda"
                if nvtx:
                    torch.cuda.nvtx.range_push("mm.task:" + name)
                try:
                    with torch.profiler.record_function("mm.task:" + name):
                        return run()
                finally:
                    if nvtx:
                        torch.cuda.nvtx.range_pop()
            return run()

        def run():
            if side is None:
                return run_on_current_stream()
            with torch.cuda.stream(side):
                return run_on_current_stream()

        def run_on_current_stream():
            dctx.device_start = dev_start
            dctx.mesh_dims = mesh_dims
            dctx.key_prefix = (self._cur_step, k)
            root_tiles = self._cur_roots
            dctx.stream_kind = kind
            if dctx.torch_device.type == "cuda":
                torch.cuda.set_device(dctx.torch_device)
            if arrival:
                # tiles that a message on the side stream delivers: wait for them on the stream
                for key in in_keys:
                    ev = arrival.pop(key, None)
                    if ev is not None:
                        torch.cuda.current_stream().wait_event(ev)
            # inputs read for the last time here are handed over: the program frees each one
            # right after its last use instead of keeping it alive for the whole task
            if self._lifetimes:
                for s in in_ids:
                    self._check_owner(s, d, f"task {name}")
            ins = [tiles[s].pop(d) if s in dying else tiles[s][d] for s in in_ids]
            if side is not None:
                for t_in in ins:            # allocated on another stream: keep its memory until this one is done
                    t_in.record_stream(side)
            for s, t_in, want in zip(in_ids, ins, in_shapes):
                if tuple(t_in.shape) != want:
                    raise RuntimeError(f"task {name}: store {s} ({stores[s]['shape']['key']}) holds a tile of shape "
                                       f"{tuple(t_in.shape)} on device {d}, expected {want}")
            if native is not None and (op["template"], d) not in self._native_off:
                try:
                    return run_native(ins)
                except torch.cuda.OutOfMemoryError:
                    # The outputs are allocated before anything is launched; when the device
                    # cannot supply them, this template goes back to the interpreted program,
                    # which allocates one output at a time as the task proceeds.
                    self._native_off.add((op["template"], d))
                    self._native_why[op["template"]] = (f"{native.out_block_bytes >> 20} MiB of outputs could not be "
                                                        "allocated")
                    torch.cuda.empty_cache()
            accs = [tiles[s].get(d) if m == 2 else None for s, m in zip(out_ids, modes)] if fused else None
            if self._lifetimes:
                # inputs read for the last time leave the tile table while the program still reads them
                held = [t.untyped_storage().data_ptr() for t in ins if isinstance(t, torch.Tensor)]
                with self._in_use_lock:
                    for ptr in held:
                        self._in_use[ptr] = self._in_use.get(ptr, 0) + 1
                try:
                    outs = prog.run(dctx, scalars, ins, accs)
                finally:
                    with self._in_use_lock:
                        for ptr in held:
                            if self._in_use[ptr] == 1:
                                del self._in_use[ptr]
                            else:
                                self._in_use[ptr] -= 1
            else:
                outs = prog.run(dctx, scalars, ins, accs)
            for oi, (s, o, m) in enumerate(zip(out_ids, outs, modes)):
                old_tile = tiles[s].get(d) if self._lifetimes else None
                if m and fused.get(oi):
                    tiles[s][d] = o          # the kernel wrote / accumulated into the accumulator itself
                elif m == 2:
                    K.accumulate_(tiles[s][d], o)
                elif m == 1:
                    tiles[s][d] = o.to(acc_dtypes[oi], copy=True)
                else:
                    tiles[s][d] = o
                if self._lifetimes:
                    self._took_buffer(s, d, old_tile, tiles[s][d])
                if side is not None and isinstance(tiles[s][d], torch.Tensor) and tiles[s][d].is_cuda:
                    tiles[s][d].record_stream(torch.cuda.default_stream(dctx.torch_device) if self._compute_stream is None
                                              else self._compute_stream)
                if s in root_tiles:
                    root_tiles[s][d] = tiles[s][d]

        native = self._native.get((op["template"], any(m == 2 for m in modes)))
        scratch_base = self._scratch_base.get(d, 0)

        def run_native(ins):
            """The task as one call into the C++ launcher: slots = input tiles, the output block,
            the scratch tile, the accumulators this launch adds into."""
            root_tiles = self._cur_roots
            blocks = [torch.empty(nb, dtype=torch.uint8, device=dctx.torch_device) for nb in native.out_chunks]
            bases = [t.data_ptr() for t in ins]
            bases.append(blocks[0].data_ptr() if blocks else 0)
            bases.append(scratch_base)
            for pos in native.acc_positions:
                bases.append(tiles[out_ids[pos]][d].data_ptr())
            ext_tiles = [self._peer_reshard.claim_source(self._direct_key[out_ids[pos]], d) for pos in native.external]
            bases.extend(t.data_ptr() for t in ext_tiles)
            bases.extend(b_.data_ptr() for b_ in blocks[1:])
            native.kernel.launch(bases, scalars, torch.cuda.current_stream().cuda_stream)
            K._count(native.num_calls)
            self.native_launches += 1
            for pos, (spec, s) in enumerate(zip(native.outputs, out_ids)):
                if spec[0] == "acc":
                    o = tiles[s][d]
                elif spec[0] == "block":
                    _, chunk, off, shape, dtype = spec
                    n = dtype.itemsize
                    for e in shape:
                        n *= e
                    o = blocks[chunk][off:off + n].view(dtype).view(shape)
                elif spec[0] == "ext":
                    o = ext_tiles[spec[1]].view(spec[2])
                elif spec[0] == "slice":
                    o = ins[spec[1]].narrow(0, scalars[0], spec[2][0]).view(spec[2])
                else:
                    o = ins[spec[1]].view(spec[2])
                if self._lifetimes:
                    self._took_buffer(s, d, tiles[s].get(d), o)
                tiles[s][d] = o
                if side is not None and o.is_cuda and self._compute_stream is not None:
                    o.record_stream(self._compute_stream)
                if s in root_tiles:
                    root_tiles[s][d] = o

        return reads, writes, body, kind

    # ------------------------------------------------------------------ reshards
    def _reshard_plan(self, src_sid: int, dst_sid: int) -> dict:
        from .. import _mm_C
        key = (src_sid, dst_sid)
        if key not in self._reshard_plans:
            self._reshard_plans[key] = _mm_C.plan_reshard(self.plan["stores"][src_sid]["shape"],
                                                          self.plan["stores"][dst_sid]["shape"])
        return self._reshard_plans[key]

    def _submit_reshard(self, k: int, op: dict, step: int, root_tiles):
        entries = self._reshard_entries.get(k)
        if entries is None:
            entries = self._reshard_entries[k] = self._make_reshard_entries(op)
        for d, reads, writes, body, label in entries:
            self.launches += 1
            if self._cuda_ctx:
                self.context.reshard(d, reads, writes, body, label, step, 1)
            else:
                self.context.reshard(d, reads, writes, body, label, step)

    def _make_reshard_entries(self, op: dict) -> list:
        """One (device, reads, writes, body, label) per local device that sends or receives a part
        of this reshard; built at the first submission, the same in every step."""
        from ..parallel.reshard import run_reshard_local, run_reshard_dist
        topo = self.topology
        src_sid, dst_sid = op["src_store"], op["dst_store"]
        rplan = self._reshard_plan(src_sid, dst_sid)
        src_shape = self.plan["stores"][src_sid]["shape"]
        dst_shape = self.plan["stores"][dst_sid]["shape"]
        buf = self.buffer_of
        tiles = self.tiles
        label = f"reshard S{src_sid}->S{dst_sid}"
        entries = []
        for d in range(op["device_start"], op["device_start"] + op["num_devices"]):
            if not topo.is_local(d):
                continue
            mine_dst = [c for c in rplan["chunks"] if c["dst_device"] == d]
            mine_src = [c for c in rplan["chunks"] if c["src_device"] == d]
            if not mine_dst and not mine_src:
                continue
            if topo.kind == "dist":
                reads = [(buf[src_sid], d)] if mine_src else []
                writes = [(buf[dst_sid], d)] if mine_dst else []
                both = mine_src + [c for c in mine_dst if c not in mine_src]

                def move(side, d=d, mine_dst=mine_dst, mine_src=mine_src, both=both):
                    root_tiles = self._cur_roots
                    prev = self._arrival.get((buf[src_sid], d))
                    if prev is not None:     # the source itself arrived by message
                        torch.cuda.current_stream().wait_event(prev)
                    pr = self._peer_reshard
                    key = (buf[src_sid], buf[dst_sid])
                    if self._lifetimes and mine_src:
                        self._check_owner(src_sid, d, label)
                    src_tile = tiles[src_sid].get(d)
                    if side is not None and src_tile is not None and src_tile.is_cuda:
                        src_tile.record_stream(side)
                    if pr is not None and pr.slots.get(key) is not None:
                        out, ev = pr.run(key, d, src_tile, both, src_shape, dst_shape, self._comm_stream(d))
                    else:
                        out, ev = run_reshard_dist(topo, d, src_tile, mine_src, mine_dst, dst_shape,
                                                   self._comm_stream(d))
                    if ev is not None and out is not None:
                        self._arrival[(buf[dst_sid], d)] = ev
                    if out is not None:
                        if side is not None and self._compute_stream is not None:
                            out.record_stream(self._compute_stream)   # allocated here, read by tasks of the compute stream
                        if self._lifetimes:
                            self._took_buffer(dst_sid, d, tiles[dst_sid].get(d), out)
                        tiles[dst_sid][d] = out
                        if dst_sid in root_tiles:
                            root_tiles[dst_sid][d] = out

                def inner(move=move):
                    side = self._streams.get(1) if self._cuda_ctx else None
                    if side is None:
                        return move(None)
                    with torch.cuda.stream(side):       # the context ordered this stream behind the producer
                        return move(side)
            else:
                if not mine_dst:
                    continue
                reads = sorted({(buf[src_sid], c["src_device"]) for c in mine_dst})
                writes = [(buf[dst_sid], d)]

                def inner(d=d, mine_dst=mine_dst):
                    root_tiles = self._cur_roots
                    if self._lifetimes:
                        for c in mine_dst:
                            self._check_owner(src_sid, c["src_device"], label)
                    out = run_reshard_local(topo, d, tiles[src_sid], mine_dst, dst_shape)
                    if self._lifetimes:
                        self._took_buffer(dst_sid, d, tiles[dst_sid].get(d), out)
                    tiles[dst_sid][d] = out
                    if dst_sid in root_tiles:
                        root_tiles[dst_sid][d] = out

            def body(inner=inner):
                if state.knobs["task_ranges"]:
                    with torch.profiler.record_function("mm." + label.replace(" ", ":", 1)):
                        return inner()
                return inner()

            entries.append((d, reads, writes, body, label))
        return entries

    # ------------------------------------------------------------------ misc
    def _check_kernel_status(self, block: bool) -> None:
        """Raises :class:`StepFailed` when a kernel of an earlier step recorded an expired bounded
        wait or an overflow in its device's status word. Without ``block`` only status copies that
        have already arrived on the host are looked at (the stream is never stalled); with it the
        device is synchronised first, so every queued step is covered."""
        for d, probe in self._probes.items():
            if block:
                with torch.cuda.device(probe.device):
                    probe.record()      # covers whatever was queued after the step's own probe
            code = probe.poll(block)
            if code:
                raise StepFailed(f"{self.name}: kernel status {code} on device {d}: "
                                 f"{K.STATUS_NAMES.get(code, 'unknown code')}")

    def wait(self):
        """Blocks until every submitted task has run and the devices are idle; raises
        :class:`StepFailed` if a task or a kernel reported an error."""
        status, msg = self.context.wait_all()
        if int(status) != 0:
            self.context.reset_error()
            raise StepFailed(f"{self.name}: {status.name}: {msg}")
        self._check_kernel_status(block=True)

    def event_log(self):
        return self.context.event_log()

    def shutdown(self):
        self.context.shutdown()
