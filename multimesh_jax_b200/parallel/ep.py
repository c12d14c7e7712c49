"""Expert parallelism over peer-mapped memory (one process per GPU).

``PeerMoE`` drives the fused router + dispatch kernel and the combine kernel of
``csrc/kernels/moe.cu`` for one expert-parallel group: token rows go straight from the kernel
that routes them into the receive region of the GPU that owns the chosen expert (no all-to-all
collective, no permuted staging copy), the local experts run on the tcgen05 GEMM kernels over
the rows that arrived, and every token pulls its results back from the owners' buffers while
weighting them with its gates. Two flag barriers per call order the phases between the GPUs
(bounded waits; the regions are double-buffered by call, which makes a third one unnecessary); the row counts of the local experts stay on the device (the expert GEMMs read them when
they start), so a call has no host synchronisation.
"""
from __future__ import annotations

from ctypes import c_int, c_int64, c_void_p
from typing import Dict, List, Sequence, Tuple

import torch

from ..ops import _lib
from ..ops import kernels as K
from . import symm

_lib.register("mm_moe_route_dispatch", c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                               c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
_lib.register("mm_moe_combine", c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_int, c_int, c_void_p])


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class PeerMoE:
    """Buffers, counters and flags of one expert-parallel group (``ranks`` are global ranks)."""

    def __init__(self, arena: symm.SymmetricArena, ranks: Sequence[int], tokens: int, d_model: int, n_experts: int):
        self.arena, self.ranks = arena, list(ranks)
        self.n = len(self.ranks)
        self.me = self.ranks.index(arena.rank)
        self.T, self.D, self.E = tokens, d_model, n_experts
        self.E_l = n_experts // self.n
        self.capacity = self.n * tokens            # a token picks an expert at most once
        shape = (self.E_l, self.capacity, d_model)
        # Two sets of regions, used alternately: the dispatch of call c+1 writes into the set that
        # nobody reads any more (its last readers, the combines of call c-1, lie behind two barriers
        # of call c), so no barrier is needed between the combine of one call and the dispatch of
        # the next - two barriers per call instead of three.
        self._sets = [{name: arena.alloc(shape, torch.bfloat16) for name in ("recv_x", "recv_o", "out", "dx")}
                      for _ in range(2)]
        self.counter = arena.alloc((max(self.E_l, 4),), torch.int32)
        self.counter.peer(arena.rank).zero_()
        self.flag_off = [arena.alloc_flag() for _ in self.ranks]   # one flag per group member
        self.epoch = 0
        self.lib = arena.lib
        self.calls = 0
        # MM_MOE_HOST_COUNTS=1: read the per-expert row counts on the host and launch exact-size
        # GEMMs (one host synchronisation per call); default: the GEMMs read the counts themselves.
        # The device-side form needs receive regions whose row count suits the CTA-pair kernel.
        import os
        self.host_counts = os.environ.get("MM_MOE_HOST_COUNTS", "0") == "1" or self.capacity < 256
        torch.cuda.synchronize()

    @staticmethod
    def required_bytes(tokens: int, d_model: int, n_experts: int) -> int:
        return 2 * 4 * n_experts * tokens * d_model * 2 + (1 << 20)

    # the regions of the current call
    recv_x = property(lambda self: self._sets[self.calls & 1]["recv_x"])
    recv_o = property(lambda self: self._sets[self.calls & 1]["recv_o"])
    out = property(lambda self: self._sets[self.calls & 1]["out"])
    dx = property(lambda self: self._sets[self.calls & 1]["dx"])

    # ------------------------------------------------------------------
    def _ptrs(self, t: symm.SymmetricTensor):
        return (c_int64 * self.n)(*[t.ptr(r) for r in self.ranks])

    def barrier(self) -> None:
        """All earlier work of every member's stream has completed (stream-ordered on each GPU)."""
        self.epoch += 1
        a = self.arena
        peers = [r for r in self.ranks if r != a.rank]
        symm.set_flags(a, [a.flag_ptr(r, self.flag_off[self.me]) for r in peers], self.epoch)
        symm.wait_flags(a, [a.flag_ptr(a.rank, self.flag_off[self.ranks.index(r)]) for r in peers], self.epoch)

    def _route_dispatch(self, x2, wr, other):
        T, D = x2.shape
        k = self.k
        dev = x2.device
        idx = torch.empty((T, k), dtype=torch.int32, device=dev)
        gates = torch.empty((T, k), dtype=torch.float32, device=dev)
        slot = torch.empty((T, k), dtype=torch.int32, device=dev)
        rc = self.lib.mm_moe_route_dispatch(x2.data_ptr(), wr.data_ptr(), other.data_ptr() if other is not None else None,
                                            T, D, self.E, k, self.E_l, self.capacity, self._ptrs(self.recv_x),
                                            self._ptrs(self.recv_o) if other is not None else None,
                                            self._ptrs(self.counter), self.n, idx.data_ptr(), gates.data_ptr(),
                                            slot.data_ptr(), _stream())
        _lib.check(rc, "mm_moe_route_dispatch")
        K._count()
        return idx, gates, slot

    def _counts(self) -> List[int]:
        local = self.counter.peer(self.arena.rank)
        counts = [int(c) for c in local[:self.E_l].tolist()]      # host synchronisation (MM_MOE_HOST_COUNTS=1 only)
        local.zero_()
        if max(counts) > self.capacity:
            raise RuntimeError("expert receive region overflowed")
        return counts

    def _device_counts(self) -> torch.Tensor:
        """Row counts of the local experts as a device tensor of their own (the counter words
        are reset for the next call): the expert GEMMs read them when they start, the host
        never does. An overflow of a receive region cannot happen (capacity = every token of
        every member) and would be reported by the dispatch kernel through the status word."""
        local = self.counter.peer(self.arena.rank)
        snap = local[:max(self.E_l, 1)].clone()
        local.zero_()
        return snap

    def _combine(self, buf, idx, slot, gates, other, dots, y, T):
        rc = self.lib.mm_moe_combine(self._ptrs(buf), self.n, idx.data_ptr(), slot.data_ptr(),
                                     gates.data_ptr() if gates is not None else None,
                                     other.data_ptr() if other is not None else None,
                                     dots.data_ptr() if dots is not None else None,
                                     y.data_ptr() if y is not None else None, T, self.D, self.k, self.E_l, self.capacity,
                                     _stream())
        _lib.check(rc, "mm_moe_combine")
        K._count()

    # ------------------------------------------------------------------
    def forward(self, x2: torch.Tensor, wr: torch.Tensor, wgu: torch.Tensor, wdown: torch.Tensor, top_k: int):
        from ..ops.moe import _expert_fwd
        self.k = top_k
        self.calls += 1
        T, me = x2.shape[0], self.arena.rank
        idx, gates, slot = self._route_dispatch(x2.contiguous(), wr.contiguous(), None)
        self.barrier()
        rx, out = self.recv_x.peer(me), self.out.peer(me)
        if self.host_counts:
            for e, m in enumerate(self._counts()):
                if m:
                    _expert_fwd(rx[e, :m], wgu[e], wdown[e], out=out[e, :m])
        else:
            counts = self._device_counts()
            for e in range(self.E_l):
                _expert_fwd(rx[e], wgu[e], wdown[e], out=out[e], count=counts[e:e + 1])
        self.barrier()
        y = torch.empty_like(x2)
        self._combine(self.out, idx, slot, gates, None, None, y, T)
        return y

    def backward(self, dy2, x2, wr, wgu, wdown, top_k: int):
        from ..ops.moe import _expert_bwd, _router_bwd
        self.k = top_k
        self.calls += 1
        T, me = x2.shape[0], self.arena.rank
        dy2 = dy2.contiguous()
        idx, gates, slot = self._route_dispatch(x2.contiguous(), wr.contiguous(), dy2)
        self.barrier()
        rx, ro, out, dxb = (t.peer(me) for t in (self.recv_x, self.recv_o, self.out, self.dx))
        dwgu = torch.zeros(wgu.shape, dtype=torch.float32, device=x2.device)
        dwdown = torch.zeros(wdown.shape, dtype=torch.float32, device=x2.device)
        if self.host_counts:
            for e, m in enumerate(self._counts()):
                if m:
                    _, dwgu_e, dwdown_e, _ = _expert_bwd(rx[e, :m], ro[e, :m], wgu[e], wdown[e], dx_out=dxb[e, :m], out=out[e, :m])
                    dwgu[e] = dwgu_e
                    dwdown[e] = dwdown_e
        else:
            counts = self._device_counts()
            for e in range(self.E_l):
                _expert_bwd(rx[e], ro[e], wgu[e], wdown[e], dx_out=dxb[e], out=out[e], count=counts[e:e + 1],
                            dwgu_out=dwgu[e], dwdown_out=dwdown[e])
        self.barrier()
        dx = torch.empty_like(x2)
        self._combine(self.dx, idx, slot, None, None, None, dx, T)
        dgates = torch.empty((T, top_k), dtype=torch.float32, device=x2.device)
        self._combine(self.out, idx, slot, None, dy2, dgates, None, T)
        dx_r, dwr = _router_bwd(x2, wr, idx.long(), gates, dgates)
        dx = (dx.float() + dx_r).to(x2.dtype)
        return dx, dwr.to(wr.dtype), dwgu.to(wgu.dtype), dwdown.to(wdown.dtype)


class PeerMoERegistry:
    """Lazily created :class:`PeerMoE` objects, one per (group, shape), from one arena."""

    def __init__(self, arena: symm.SymmetricArena):
        self.arena = arena
        self._ops: Dict[Tuple, PeerMoE] = {}

    def get(self, ranks: Tuple[int, ...], tokens: int, d_model: int, n_experts: int) -> PeerMoE:
        key = (tuple(ranks), tokens, d_model, n_experts)
        if key not in self._ops:
            self._ops[key] = PeerMoE(self.arena, ranks, tokens, d_model, n_experts)
        return self._ops[key]
