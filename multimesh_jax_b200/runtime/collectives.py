"""Device topology and in-task collectives.

A compiled step addresses ``num_devices`` devices by ordinal. Three kinds of
topology carry them:

* ``cpu``  - every ordinal is a *virtual* CPU device of this process (the
  stand-in for GPUs that the reference gets from
  ``--xla_force_host_platform_device_count``); collectives are rendezvous
  between the runtime's worker threads.
* ``cuda`` - every ordinal is a CUDA device of this process.
* ``dist`` - one process per device (``torch.distributed``; NCCL on GPUs,
  gloo on CPUs): ordinal ``r`` lives in rank ``r``; collectives are
  ``torch.distributed`` calls on sub-groups created once per device list.
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional, Sequence, Tuple

import torch


class Topology:
    def __init__(self, kind: str, num_devices: int, rank: int = 0, device: Optional[torch.device] = None):
        assert kind in ("cpu", "cuda", "dist")
        self.kind = kind
        self.num_devices = num_devices
        self.rank = rank
        self._dist_device = device
        if kind == "dist":
            self.local_devices = [rank]
        else:
            self.local_devices = list(range(num_devices))
        self._groups: Dict[Tuple[int, ...], object] = {}

    @staticmethod
    def auto(num_devices: int, backend: Optional[str] = None) -> "Topology":
        import torch.distributed as dist
        if backend in (None, "dist") and dist.is_available() and dist.is_initialized() and \
                dist.get_world_size() >= num_devices and (backend == "dist" or num_devices > 1 or dist.get_world_size() == 1):
            if backend == "dist" or dist.get_world_size() == num_devices:
                dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
                return Topology("dist", num_devices, rank=dist.get_rank(), device=dev)
        if backend in (None, "cuda") and torch.cuda.is_available() and torch.cuda.device_count() >= num_devices:
            return Topology("cuda", num_devices)
        if backend == "cuda":
            raise RuntimeError(f"backend 'cuda' needs {num_devices} CUDA devices in this process")
        return Topology("cpu", num_devices)

    def torch_device(self, ordinal: int) -> torch.device:
        if self.kind == "cpu":
            return torch.device("cpu")
        if self.kind == "cuda":
            return torch.device("cuda", ordinal)
        return self._dist_device

    def is_local(self, ordinal: int) -> bool:
        return ordinal in self.local_devices

    def process_group(self, ranks: Sequence[int]):
        """The ``torch.distributed`` group of ``ranks`` (created collectively on
        first use: every rank must ask for the same groups in the same order)."""
        import torch.distributed as dist
        key = tuple(ranks)
        if key not in self._groups:
            if len(key) == dist.get_world_size():
                self._groups[key] = dist.group.WORLD
            else:
                self._groups[key] = dist.new_group(list(key))
        return self._groups[key]

    def prepare_groups(self, meshes: Sequence[Tuple[int, Sequence[int]]]) -> None:
        """Create, on every rank and in one global order, the process groups that tasks on the
        meshes ``(device_start, mesh_dims)`` can ask for: one per non-empty subset of mesh axes
        and per position along the other axes. ``torch.distributed.new_group`` is collective
        over the whole job, so groups cannot be made lazily by the ranks that happen to need
        them (two pipeline stages would each make "their" tensor-parallel group first)."""
        if self.kind != "dist":
            return
        import itertools
        wanted = set()
        for start, dims in meshes:
            n = 1
            for s in dims:
                n *= s
            axes_all = [a for a, s in enumerate(dims) if s > 1]
            for r in range(1, len(axes_all) + 1):
                for axes in itertools.combinations(axes_all, r):
                    for o in range(n):
                        wanted.add(tuple(start + g for g in mesh_group(o, dims, list(axes))))
        for key in sorted(wanted):
            if len(key) > 1:
                self.process_group(key)


class Rendezvous:
    """Exchange of one object per participant between threads of a process."""

    def __init__(self):
        self._cv = threading.Condition()
        self._slots: Dict[object, Dict[int, object]] = {}
        self._taken: Dict[object, int] = {}
        self.timeout_s = 120.0

    def exchange(self, key, group: Sequence[int], me: int, obj) -> List[object]:
        with self._cv:
            slot = self._slots.setdefault(key, {})
            slot[me] = obj
            self._cv.notify_all()
            ok = self._cv.wait_for(lambda: len(slot) == len(group), timeout=self.timeout_s)
            if not ok:
                raise TimeoutError(f"collective {key!r}: only {len(slot)} of {len(group)} participants arrived")
            out = [slot[r] for r in group]
            self._taken[key] = self._taken.get(key, 0) + 1
            if self._taken[key] == len(group):
                del self._slots[key]
                del self._taken[key]
            return out


class FusedTP:
    """Lazily created fused GEMM+all-reduce operators, one per tensor-parallel rank group,
    all carved out of one symmetric arena that is created collectively up front."""

    def __init__(self, arena):
        self.arena = arena
        self._ops: Dict[Tuple[int, ...], object] = {}

    def get(self, ranks: Tuple[int, ...]):
        from ..parallel.tp import FusedLinearAllReduce
        if ranks not in self._ops:
            self._ops[ranks] = FusedLinearAllReduce(self.arena, ranks)
        return self._ops[ranks]

    def get_scatter(self, ranks: Tuple[int, ...]):
        """GEMM -> reduce-scatter operator of a group (its members create it at the same point of
        the same program, so the arena offsets agree)."""
        from ..parallel.tp import FusedLinearReduceScatter
        key = ("rs",) + tuple(ranks)
        if key not in self._ops:
            self._ops[key] = FusedLinearReduceScatter(self.arena, ranks)
        return self._ops[key]

    def get_gather(self, ranks: Tuple[int, ...]):
        from ..parallel.tp import FusedAllGatherLinear
        key = ("ag",) + tuple(ranks)
        if key not in self._ops:
            self._ops[key] = FusedAllGatherLinear(self.arena, ranks)
        return self._ops[key]


def mesh_group(ordinal: int, mesh_dims: Sequence[int], axes: Sequence[int]) -> List[int]:
    """Ordinals (within the task's device list) that differ from ``ordinal``
    only in the coordinates of ``axes``; row-major mesh."""
    strides = []
    acc = 1
    for s in reversed(mesh_dims):
        strides.append(acc)
        acc *= s
    strides = list(reversed(strides))
    coord = [(ordinal // st) % sz for st, sz in zip(strides, mesh_dims)]
    group = [0]
    base = sum(c * st for i, (c, st) in enumerate(zip(coord, strides)) if i not in axes)
    group = [base]
    for a in sorted(axes):
        group = [g + k * strides[a] for g in group for k in range(mesh_dims[a])]
    return sorted(group)


def tile_box(shape_dict: dict, ordinal: int) -> Tuple[List[int], List[int]]:
    from .. import _mm_C
    return _mm_C.tile_box(shape_dict, ordinal)


_LOCAL_PLANS: Dict[Tuple[str, str], Optional[Dict[int, list]]] = {}


def _local_only_chunks(src: dict, dst: dict) -> Optional[Dict[int, list]]:
    """Chunks of the reshard ``src`` -> ``dst`` per destination device when each of them comes
    from that same device's source tile; None when any piece has to cross devices."""
    key = (src["key"], dst["key"])
    if key not in _LOCAL_PLANS:
        from .. import _mm_C
        chunks = _mm_C.plan_reshard(src, dst)["chunks"]
        if all(c["src_device"] == c["dst_device"] for c in chunks):
            per: Dict[int, list] = {}
            for c in chunks:
                per.setdefault(c["dst_device"], []).append(c)
            _LOCAL_PLANS[key] = per
        else:
            _LOCAL_PLANS[key] = None
    return _LOCAL_PLANS[key]


class DeviceCtx:
    """What a task body sees of the device it runs on."""

    def __init__(self, topology: Topology, device: int, rendezvous: Rendezvous):
        self.topology = topology
        self.device = device
        self.torch_device = topology.torch_device(device)
        self.rendezvous = rendezvous
        self.fused_tp = None  # FusedTP registry (one-process-per-GPU CUDA jobs only)
        self.peer_moe = None  # PeerMoERegistry (same)
        self.peer_comm = None  # PeerCommRegistry (same): in-task all-reduce / reshard over peer memory
        # set per task launch
        self.device_start = 0
        self.mesh_dims: Sequence[int] = (1,)
        self.key_prefix: Tuple = ()
        self.stream_kind = 0      # 0 compute, 1 communication, 2 auxiliary stream of the runtime context

    # ------------------------------------------------------------------
    def _exchange(self, key, group_ordinals: List[int], tensor: torch.Tensor) -> List[torch.Tensor]:
        me = self.device - self.device_start
        topo = self.topology
        if topo.kind == "dist":
            import torch.distributed as dist
            pg = topo.process_group([self.device_start + o for o in group_ordinals])
            outs = [torch.empty_like(tensor) for _ in group_ordinals]
            dist.all_gather(outs, tensor.contiguous(), group=pg)
            return outs
        parts = self.rendezvous.exchange((self.key_prefix, key, tuple(group_ordinals)), group_ordinals, me, tensor)
        return [p.to(self.torch_device) if p.device != self.torch_device else p for p in parts]

    def group_of(self, axes: Sequence[int]) -> Tuple[List[int], int]:
        """Ordinals of the devices that differ from this one along ``axes`` only, and this
        device's position among them."""
        me = self.device - self.device_start
        group = mesh_group(me, self.mesh_dims, list(axes))
        return group, group.index(me)

    def all_to_all(self, key, group: List[int], rows: torch.Tensor, counts: List[int]
                   ) -> Tuple[torch.Tensor, List[int]]:
        """``rows`` holds, back to back, ``counts[r]`` rows for every member ``r`` of ``group``.
        Returns the rows this device receives (ordered by sender) and how many each sender sent."""
        me = self.device - self.device_start
        topo = self.topology
        if topo.kind == "dist":
            import torch.distributed as dist
            pg = topo.process_group([self.device_start + o for o in group])
            cnt = torch.tensor(counts, dtype=torch.int64, device=rows.device)
            got = torch.empty_like(cnt)
            dist.all_to_all_single(got, cnt, group=pg)
            recv_counts = [int(c) for c in got.tolist()]
            out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
            dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts, input_split_sizes=list(counts),
                                   group=pg)
            return out, recv_counts
        pieces = list(torch.split(rows, list(counts)))
        everyone = self.rendezvous.exchange((self.key_prefix, "a2a", key, tuple(group)), group, me, pieces)
        my = group.index(me)
        mine = [everyone[s][my] for s in range(len(group))]
        mine = [p.to(self.torch_device) if p.device != self.torch_device else p for p in mine]
        return torch.cat(mine, dim=0), [int(p.shape[0]) for p in mine]

    def all_reduce(self, x: torch.Tensor, axes: Sequence[int], key, in_place: bool = False) -> torch.Tensor:
        """Sum of ``x`` over the devices that differ from this one along ``axes``. With
        ``in_place`` (the planner found that nothing else reads the operand: the once-per-step
        reduction of a gradient accumulator) the result overwrites ``x``'s buffer."""
        me = self.device - self.device_start
        group = mesh_group(me, self.mesh_dims, list(axes))
        if len(group) == 1:
            return x
        if self.topology.kind == "dist":
            if self.peer_comm is not None:
                comm = self.peer_comm.get(tuple(self.device_start + o for o in group), self.stream_kind)
                if comm.supports(x):
                    return comm.all_reduce(x, out=x if in_place and x.is_contiguous() else None)
            import torch.distributed as dist
            pg = self.topology.process_group([self.device_start + o for o in group])
            out = x if in_place and x.is_contiguous() else x.contiguous().clone()
            dist.all_reduce(out, group=pg)
            return out
        parts = self._exchange(("ar", key), group, x)
        acc = parts[0].float() if x.dtype in (torch.bfloat16, torch.float16) else parts[0].clone()
        for p in parts[1:]:
            acc = acc + (p.float() if acc.dtype != p.dtype else p)
        if in_place:
            # every member has read the others' tensors (the exchange above returns after all
            # members arrived); wait for all of them to finish summing before overwriting
            self.rendezvous.exchange((self.key_prefix, "ar-done", key, tuple(group)), group, me, None)
            x.copy_(acc.to(x.dtype))
            return x
        return acc.to(x.dtype)

    def linear_all_reduce(self, x: torch.Tensor, w: torch.Tensor, axes: Sequence[int], is_dgrad: bool, key
                          ) -> torch.Tensor:
        """``all_reduce(linear(x, w))`` (or of the input gradient ``dy @ w``) over the mesh
        axes ``axes``. One-process-per-GPU jobs run the fused tcgen05 GEMM + NVLink
        all-reduce kernel; everything else computes the partial result and reduces it."""
        from ..ops import mm_ops
        me = self.device - self.device_start
        group = mesh_group(me, self.mesh_dims, list(axes))
        fused = self.fused_tp
        if fused is not None and len(group) > 1 and x.is_cuda and x.dtype == torch.bfloat16:
            ranks = tuple(self.device_start + o for o in group)
            op = fused.get(ranks)
            if is_dgrad:
                n_lead = w.dim() - 1
                w2 = w.reshape(-1, w.shape[-1])
                a2 = x.reshape(-1, w2.shape[0])
                M, N, Kd = a2.shape[0], w2.shape[1], w2.shape[0]
                if op.supported(M, N, Kd, x.dtype):
                    y = op(a2, w2, b_mn=True)
                    return y.view(*x.shape[:x.dim() - n_lead], N)
            else:
                w2 = w.reshape(-1, w.shape[-1])
                a2 = x.reshape(-1, x.shape[-1])
                M, N, Kd = a2.shape[0], w2.shape[0], a2.shape[1]
                if op.supported(M, N, Kd, x.dtype):
                    y = op(a2, w2)
                    return y.view(*x.shape[:-1], *w.shape[:-1])
        y = mm_ops.linear_dgrad_impl(x, w) if is_dgrad else mm_ops.linear_impl(x, w)
        return self.all_reduce(y, axes, key)

    def combine_softmax_stats(self, stats: torch.Tensor, targets: torch.Tensor, group: List[int], key):
        """Global softmax statistics of a vocabulary-sharded cross-entropy from this shard's
        [rows, 3] array (see ``kernels.cross_entropy_stats``): returns ([rows, 2], loss per row)."""
        from ..ops import kernels as K
        if self.topology.kind == "dist" and self.peer_comm is not None and stats.is_cuda:
            comm = self.peer_comm.get(tuple(self.device_start + o for o in group), self.stream_kind)
            ptrs = comm.share_small(stats)
            return K.cross_entropy_combine(None, targets, stat_ptrs=ptrs)
        parts = self._exchange(("ce", key), group, stats)
        return K.cross_entropy_combine(parts, targets)

    def _scatter_slice(self, full: torch.Tensor, src: dict, dst: dict) -> torch.Tensor:
        """This device's tile of layout ``dst`` cut out of its tile of the coarser layout ``src``."""
        local = _local_only_chunks(src, dst)
        if local is None:
            raise RuntimeError("reduce-scatter target is not a refinement of the source layout")
        # by position in the task's sub-mesh: the layouts name the devices the template was compiled for
        mine = local.get(src["device_start"] + self.device - self.device_start)
        if mine is None:
            raise RuntimeError(f"reduce-scatter: device {self.device} has no part in {src['key']} -> {dst['key']}")
        out = torch.empty(dst["shard_size"], dtype=full.dtype, device=full.device)
        for c in mine:
            ext = [h - l for l, h in zip(c["lo"], c["hi"])]
            s_box = tuple(slice(o, o + e) for o, e in zip(c["src_offset"], ext))
            d_box = tuple(slice(o, o + e) for o, e in zip(c["dst_offset"], ext))
            out[d_box] = full[s_box]
        return out

    def reduce_scatter(self, x: torch.Tensor, axes: Sequence[int], dim: int, src: dict, dst: dict, key) -> torch.Tensor:
        """Sum of ``x`` over the devices along ``axes``, of which this device keeps its part of
        dimension ``dim`` (layout ``dst``, a refinement of ``src``). One-process-per-GPU jobs pull
        only their own share from the peers (half of an all-reduce's traffic); elsewhere the sum
        is formed by the all-reduce and sliced."""
        me = self.device - self.device_start
        group = mesh_group(me, self.mesh_dims, list(axes))
        if len(group) == 1:
            return x
        if self.topology.kind == "dist" and self.peer_comm is not None:
            comm = self.peer_comm.get(tuple(self.device_start + o for o in group), self.stream_kind)
            if comm.supports_scatter(x, dim):
                return comm.reduce_scatter(x, dim, group.index(me))
        return self._scatter_slice(self.all_reduce(x, axes, key), src, dst)

    def linear_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, axes: Sequence[int], is_dgrad: bool, dim: int,
                              src: dict, dst: dict, key) -> torch.Tensor:
        """``reduce_scatter(linear(x, w))`` (or of the input gradient) over ``axes`` along the row
        dimension ``dim`` of the product. One-process-per-GPU jobs run the fused tcgen05 GEMM whose
        epilogue pushes each tile's partial sums to the rank that owns those rows."""
        from ..ops import mm_ops
        me = self.device - self.device_start
        group = mesh_group(me, self.mesh_dims, list(axes))
        fused = self.fused_tp
        if fused is not None and len(group) > 1 and x.is_cuda and x.dtype == torch.bfloat16:
            ranks = tuple(self.device_start + o for o in group)
            op = fused.get_scatter(ranks)
            if is_dgrad:
                w2 = w.reshape(-1, w.shape[-1])
                a2 = x.reshape(-1, w2.shape[0])
                out_shape = list(x.shape[:x.dim() - (w.dim() - 1)]) + [w2.shape[1]]
                N, Kd = w2.shape[1], w2.shape[0]
            else:
                w2 = w.reshape(-1, w.shape[-1])
                a2 = x.reshape(-1, x.shape[-1])
                out_shape = list(x.shape[:-1]) + list(w.shape[:-1])
                N, Kd = w2.shape[0], a2.shape[1]
            M = a2.shape[0]
            outer = 1
            for s_ in out_shape[:dim]:
                outer *= s_
            rows_per_outer = M // outer
            if op.supported(M, N, Kd, outer, x.dtype):
                y = op(a2, w2, b_mn=is_dgrad, outer=outer)          # [M / g, N]
                out_shape[dim] //= len(group)
                return y.view(out_shape)
        y = mm_ops.linear_dgrad_impl(x, w) if is_dgrad else mm_ops.linear_impl(x, w)
        return self.reduce_scatter(y, axes, dim, src, dst, key)

    def all_gather_linear(self, x: torch.Tensor, w: torch.Tensor, is_dgrad: bool, axes: Sequence[int], dim: int,
                          src: dict, dst: dict, key) -> Tuple[torch.Tensor, torch.Tensor]:
        """``linear(all_gather(x), w)`` for an activation whose row dimension ``dim`` is sharded
        over ``axes``; returns the product and the gathered activation. One-process-per-GPU jobs
        run the fused kernel that pulls the peers' rows while the tensor cores already work on
        the rows that have arrived."""
        from ..ops import mm_ops
        me = self.device - self.device_start
        group = mesh_group(me, self.mesh_dims, list(axes))
        fused = self.fused_tp
        if fused is not None and len(group) > 1 and x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous():
            ranks = tuple(self.device_start + o for o in group)
            op = fused.get_gather(ranks)
            outer = 1
            for s_ in x.shape[:dim]:
                outer *= s_
            a2 = x.reshape(-1, x.shape[-1])
            w2 = w.reshape(-1, w.shape[-1])
            if is_dgrad and w.dim() == 2 and op.supported(a2.shape[0], a2.shape[1], outer, x.dtype):
                y, full = op(a2, w2, b_mn=True, outer=outer)
                full_shape = list(x.shape)
                full_shape[dim] *= len(group)
                return y.view(*full_shape[:-1], w2.shape[1]), full.view(full_shape)
            if not is_dgrad and op.supported(a2.shape[0], a2.shape[1], outer, x.dtype):
                y, full = op(a2, w2, outer=outer)
                full_shape = list(x.shape)
                full_shape[dim] *= len(group)
                return y.view(*full_shape[:-1], *w.shape[:-1]), full.view(full_shape)
        full = self.spmd_reshard(x, src, dst, key)
        y = mm_ops.linear_dgrad_impl(full, w) if is_dgrad else mm_ops.linear_impl(full, w)
        return y, full

    def spmd_reshard(self, x: torch.Tensor, src: dict, dst: dict, key) -> torch.Tensor:
        """Local tile of layout ``dst`` from tiles in layout ``src`` (same
        devices): gather every tile, assemble the global array, slice."""
        n = src["num_devices"]
        me = self.device - self.device_start
        group = list(range(n))
        local = _local_only_chunks(src, dst)
        if local is not None:
            # every destination tile is made of pieces of the same device's source tile (replicated
            # -> sharded, or a coarser -> finer split): a slice, no exchange. All members take this
            # branch together because the plan depends on the two layouts only.
            # The layouts name the devices the task's template was compiled for; a task that moves
            # between sub-meshes per microbatch runs the same template elsewhere, so the chunks are
            # looked up by this device's position in the task's sub-mesh.
            mine = local.get(src["device_start"] + me)
            if mine is None:
                raise RuntimeError(f"spmd_reshard: device {self.device} (position {me}) has no part in {src['key']} -> {dst['key']}")
            out = torch.empty(dst["shard_size"], dtype=x.dtype, device=x.device)
            for c in mine:
                ext = [h - l for l, h in zip(c["lo"], c["hi"])]
                s_box = tuple(slice(o, o + e) for o, e in zip(c["src_offset"], ext))
                d_box = tuple(slice(o, o + e) for o, e in zip(c["dst_offset"], ext))
                out[d_box] = x[s_box]
            return out
        if self.topology.kind == "dist" and self.peer_comm is not None:
            comm = self.peer_comm.get(tuple(self.device_start + o for o in group), self.stream_kind)
            from ..parallel.reshard import PeerReshard
            from .. import _mm_C
            if x.is_cuda and x.numel() * x.element_size() >= comm.MIN_BYTES and \
                    PeerReshard.pullable(_mm_C.plan_reshard(src, dst), src, dst):
                return comm.reshard(x, src, dst)
        parts = self._exchange(("rs", key), group, x)
        full = torch.empty(src["sizes"], dtype=x.dtype, device=x.device)
        for o, p in zip(group, parts):
            lo, hi = tile_box(src, o)
            full[tuple(slice(a, b) for a, b in zip(lo, hi))] = p
        lo, hi = tile_box(dst, me)
        return full[tuple(slice(a, b) for a, b in zip(lo, hi))].contiguous()
