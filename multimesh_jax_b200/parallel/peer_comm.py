"""In-task collectives over peer-mapped memory (one process per GPU).

``PeerGroupComm`` serves one device group of a task (a tensor- or data-parallel group):

* ``all_reduce``  - gradient sums after the microbatch loop, partial results: every rank
  copies its tensor into a staging tile, then *pulls* its 1/g share from all members with the
  reduce-pull kernel (the reduce-scatter half: loads over NVLink, fp32 accumulation, one pass),
  then pulls the other members' reduced shares (the all-gather half). The volume per GPU is the
  ring optimum, 2 (g-1)/g of the tensor, and there is no NCCL call.
* ``reshard``     - a layout change inside the group (FSDP parameter gather before the loop,
  batch <-> hidden transposes): staging copy, then the reshard pull kernel writes the new
  layout directly from the members' tiles.

Phases are ordered between the GPUs by flag barriers with time-bounded waits; staging tiles
live in the symmetric arena, one pair per distinct size.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Dict, Optional, Sequence, Tuple

import torch

from ..ops import _lib
from ..ops import kernels as K
from . import symm

_lib.register("mm_reduce_pull", c_int, [c_void_p, c_int, c_void_p, c_int64, c_int, c_float, c_void_p])
_lib.register("mm_reduce_pull_chunked", c_int, [c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64, c_int, c_float, c_void_p])


class PeerGroupComm:
    MIN_BYTES = 256 << 10      # below this a library collective's latency wins

    def __init__(self, arena: symm.SymmetricArena, ranks: Sequence[int], stage: Dict[int, tuple]):
        self.arena, self.ranks = arena, list(ranks)
        self.g = len(self.ranks)
        self.me = self.ranks.index(arena.rank)
        self.flag_off = [arena.alloc_flag() for _ in self.ranks]
        self.epoch = 0
        # staging tiles are shared by all groups of this rank: the members of a group run the same
        # program, so they create size classes in the same order and the offsets agree
        self.stage = stage
        self.calls = 0

    # ------------------------------------------------------------------
    def barrier(self) -> None:
        self.epoch += 1
        a = self.arena
        peers = [r for r in self.ranks if r != a.rank]
        symm.set_flags(a, [a.flag_ptr(r, self.flag_off[self.me]) for r in peers], self.epoch)
        symm.wait_flags(a, [a.flag_ptr(a.rank, self.flag_off[self.ranks.index(r)]) for r in peers], self.epoch)

    def _tiles(self, nbytes: int):
        """Two staging tiles of at least ``nbytes`` (sizes are rounded up so that tensors of
        similar size share them; every member asks in the same order, so offsets agree)."""
        size = 1 << max(20, (nbytes - 1).bit_length())
        if size not in self.stage:
            self.stage[size] = (self.arena.alloc((size,), torch.uint8), self.arena.alloc((size,), torch.uint8))
        return self.stage[size]

    def supports(self, x: torch.Tensor) -> bool:
        n = x.numel() * x.element_size()
        return (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and n >= self.MIN_BYTES
                and n % (16 * self.g) == 0)

    # ------------------------------------------------------------------
    def all_reduce(self, x: torch.Tensor, scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        a, g, me = self.arena, self.g, self.me
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        s_in, s_red = self._tiles(nbytes)
        stream = torch.cuda.current_stream().cuda_stream
        K_lib = a.lib
        s_in.peer(a.rank)[:nbytes].view(x.dtype).view(x.shape).copy_(x)
        self.barrier()                                    # every member's tensor is staged
        share = nbytes // g
        srcs = (c_int64 * g)(*[s_in.ptr(r) + me * share for r in self.ranks])
        rc = K_lib.mm_reduce_pull(srcs, g, s_red.ptr(a.rank) + me * share, share, x.element_size(), scale, stream)
        _lib.check(rc, "mm_reduce_pull")
        K._count()
        self.barrier()                                    # every member's share is reduced
        if out is None:
            out = torch.empty_like(x)                     # else in place: x was staged above, its buffer is free
        for i, r in enumerate(self.ranks):                # all-gather half: pull each owner's share
            one = (c_int64 * 1)(s_red.ptr(r) + i * share)
            rc = K_lib.mm_reduce_pull(one, 1, out.data_ptr() + i * share, share, x.element_size(), 1.0, stream)
            _lib.check(rc, "mm_reduce_pull")
            K._count()
        self.barrier()                                    # staging tiles may be overwritten again
        self.calls += 1
        return out

    SMALL_BYTES = 1 << 20

    def share_small(self, x: torch.Tensor):
        """Makes a small tensor (statistics, counts; at most ``SMALL_BYTES``) readable by the
        group: copies it into this rank's slot of a double-buffered symmetric tile and passes a
        flag barrier. Returns the device addresses of every member's copy, in group order; they
        stay valid until this rank's next call but one."""
        a = self.arena
        nbytes = x.numel() * x.element_size()
        if nbytes > self.SMALL_BYTES:
            raise ValueError("share_small is for small tensors")
        if not hasattr(self, "_small"):
            self._small = [a.alloc((self.SMALL_BYTES,), torch.uint8) for _ in range(2)]
            self._small_calls = 0
        self._small_calls += 1
        buf = self._small[self._small_calls & 1]
        buf.peer(a.rank)[:nbytes].view(x.dtype).view(x.shape).copy_(x)
        self.barrier()
        return [buf.ptr(r) for r in self.ranks]

    def supports_scatter(self, x: torch.Tensor, dim: int) -> bool:
        """Reduce-scatter along ``dim`` as a pull of this rank's share: the share of every outer
        index must be a whole number of 16-byte vectors."""
        if not (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.is_contiguous()):
            return False
        if x.numel() * x.element_size() < self.MIN_BYTES or dim >= x.dim() or x.shape[dim] % self.g:
            return False
        inner = x.element_size() * (x.shape[dim] // self.g)
        for s_ in x.shape[dim + 1:]:
            inner *= s_
        return inner % 16 == 0

    def reduce_scatter(self, x: torch.Tensor, dim: int, index: int, scale: float = 1.0) -> torch.Tensor:
        """Sum of the members' ``x`` restricted to part ``index`` (of ``g``) of dimension ``dim``:
        staging copy, one barrier, one pull kernel that reads only this rank's share from every
        member (a (g-1)/g-th of the tensor crosses NVLink into this GPU), one barrier."""
        a, g = self.arena, self.g
        nbytes = x.numel() * x.element_size()
        s_in, _ = self._tiles(nbytes)
        s_in.peer(a.rank)[:nbytes].view(x.dtype).view(x.shape).copy_(x)
        self.barrier()
        outer = 1
        for s_ in x.shape[:dim]:
            outer *= s_
        stride = nbytes // outer                      # bytes of one outer index in the source
        chunk = stride // g                           # this rank's share of it
        out_shape = list(x.shape)
        out_shape[dim] //= g
        out = torch.empty(out_shape, dtype=x.dtype, device=x.device)
        srcs = (c_int64 * g)(*[s_in.ptr(r) + index * chunk for r in self.ranks])
        rc = a.lib.mm_reduce_pull_chunked(srcs, g, out.data_ptr(), chunk, outer, stride, x.element_size(), scale,
                                          torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "mm_reduce_pull_chunked")
        K._count()
        self.barrier()                                # staging tiles may be overwritten again
        self.calls += 1
        return out

    def reshard(self, x: torch.Tensor, src: dict, dst: dict) -> torch.Tensor:
        """Local tile in layout ``dst`` from the members' tiles in layout ``src`` (layouts over
        exactly this group's devices)."""
        from .. import _mm_C
        from ..compiler.capture import DTYPE_FROM_NAME
        a = self.arena
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        s_in, _ = self._tiles(nbytes)
        s_in.peer(a.rank)[:nbytes].view(x.dtype).view(x.shape).copy_(x)
        self.barrier()
        plan = _mm_C.plan_reshard(src, dst)
        d = src["device_start"] + self.me
        mine = [c for c in plan["chunks"] if c["dst_device"] == d]
        out = torch.empty(dst["shard_size"], dtype=DTYPE_FROM_NAME[dst["dtype"]], device=x.device)
        start = src["device_start"]
        recs = symm.build_pull_chunks(mine, list(src["shard_size"]), list(dst["shard_size"]),
                                      lambda dev: s_in.ptr(self.ranks[dev - start]), out.data_ptr(), x.element_size())
        for i in range(0, len(recs), 64):
            symm.reshard_pull(recs[i:i + 64], x.element_size(), a)
        self.barrier()
        self.calls += 1
        return out


class PeerCommRegistry:
    def __init__(self, arena: symm.SymmetricArena):
        self.arena = arena
        self._ops: Dict[Tuple[int, ...], PeerGroupComm] = {}
        self._stage: Dict[int, Dict[int, tuple]] = {}     # stream kind -> size class -> staging pair

    def get(self, ranks: Tuple[int, ...], stream_kind: int = 0) -> PeerGroupComm:
        """The group's communicator for tasks of one stream kind. Collectives queued on different
        streams can overlap on the GPU, so each kind gets its own flags, epochs and staging tiles;
        the members of a group ask in the same program order, so the arena offsets agree."""
        key = (tuple(ranks), stream_kind)
        if key not in self._ops:
            self._ops[key] = PeerGroupComm(self.arena, ranks, self._stage.setdefault(stream_kind, {}))
        return self._ops[key]
