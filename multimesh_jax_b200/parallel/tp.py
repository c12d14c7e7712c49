"""Tensor-parallel linear layers fused with their all-reduce.

``FusedLinearAllReduce`` drives ``mm_gemm_allreduce_bf16``: the tcgen05 GEMM whose
epilogue pushes every finished tile to the peers' receive buffers over NVLink and adds
the tiles it receives, so the reduction overlaps the matrix multiply tile by tile and no
separate collective is launched. Receive buffers and flags live in the symmetric arena
(:mod:`multimesh_jax_b200.parallel.symm`); they are double-buffered by call parity and the
flags carry an epoch, so nothing is ever reset between calls.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int64, c_void_p
from typing import Dict, Sequence, Tuple

import torch

from ..ops import _lib
from ..ops import kernels as K
from . import symm

_lib.register("mm_gemm_allreduce_bf16", c_int, [c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_void_p, c_int64,
                                                c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                c_int, c_void_p])

BM, BN = 128, 256


class _BufferSet:
    def __init__(self, arena: symm.SymmetricArena, M: int, N: int, npeers: int):
        self.tiles = 4 * ((M + BM - 1) // BM) * ((N + BN - 1) // BN)   # one flag per 32-row quarter of a tile
        self.recv = [arena.alloc((npeers, M, N), torch.bfloat16) for _ in range(2)]
        self.flags = [arena.alloc((npeers, self.tiles), torch.int32) for _ in range(2)]
        self.epoch = 0


class FusedLinearAllReduce:
    """One instance per tensor-parallel group (``ranks`` are global ranks, this rank included)."""

    def __init__(self, arena: symm.SymmetricArena, ranks: Sequence[int]):
        self.arena = arena
        self.ranks = list(ranks)
        self.rank = arena.rank
        self.peers = [r for r in self.ranks if r != self.rank]
        self.sets: Dict[Tuple[int, int], _BufferSet] = {}
        self.lib = _lib.load()
        self.calls = 0

    def _slot_in(self, peer: int) -> int:
        """Index of this rank among ``peer``'s peers."""
        others = [r for r in self.ranks if r != peer]
        return others.index(self.rank)

    def __call__(self, a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False) -> torch.Tensor:
        """all_reduce(A[M,K] @ B[N,K]^T) with this rank's K-shard of both operands."""
        M, Kd = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
        N = b.shape[1] if b_mn else b.shape[0]
        key = (M, N)
        bs = self.sets.get(key)
        if bs is None:
            bs = self.sets[key] = _BufferSet(self.arena, M, N, len(self.peers))
        bs.epoch += 1
        par = bs.epoch & 1
        recv, flags = bs.recv[par], bs.flags[par]
        npeers = len(self.peers)
        esz_tile = M * N * 2
        recv_local = (c_int64 * npeers)(*[recv.ptr(self.rank) + i * esz_tile for i in range(npeers)])
        flag_local = (c_int64 * npeers)(*[flags.ptr(self.rank) + i * bs.tiles * 4 for i in range(npeers)])
        recv_peer = (c_int64 * npeers)(*[recv.ptr(p) + self._slot_in(p) * esz_tile for p in self.peers])
        flag_peer = (c_int64 * npeers)(*[flags.ptr(p) + self._slot_in(p) * bs.tiles * 4 for p in self.peers])
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        rc = self.lib.mm_gemm_allreduce_bf16(a.data_ptr(), int(a_mn), a.stride(0), b.data_ptr(), int(b_mn), b.stride(0),
                                             out.data_ptr(), out.stride(0), M, N, Kd, recv_local, recv_peer,
                                             flag_local, flag_peer, npeers, bs.epoch,
                                             torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "mm_gemm_allreduce_bf16")
        K._count()
        self.calls += 1
        return out

    @staticmethod
    def supported(M: int, N: int, Kd: int, dtype: torch.dtype) -> bool:
        return dtype == torch.bfloat16 and N % 32 == 0 and Kd % 8 == 0


_lib.register("mm_gemm_reducescatter_bf16", c_int, [c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_void_p, c_int64,
                                                    c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                    c_int, c_int, c_int, c_void_p])


class _ScatterBufferSet:
    def __init__(self, arena: symm.SymmetricArena, Ms: int, N: int, g: int):
        self.tiles = 4 * ((Ms + BM - 1) // BM) * ((N + BN - 1) // BN)   # one flag per 32-row quarter of a shard tile
        self.recv = [arena.alloc((g - 1, Ms, N), torch.bfloat16) for _ in range(2)]
        self.flags = [arena.alloc((g - 1, self.tiles), torch.int32) for _ in range(2)]
        self.epoch = 0
        self.args = [None, None]      # per parity: the four address arrays of a call (they never change)


class FusedLinearReduceScatter:
    """``reduce_scatter(A @ B^T)`` over one tensor-parallel group with this rank's K-shard of
    both operands (``mm_gemm_reducescatter_bf16``): the tcgen05 GEMM whose epilogue pushes the
    partial sums of every tile to the rank that owns those rows and adds what it receives for
    its own rows. Rows are owned in chunks (``outer`` chunks per rank: ``outer`` = 1 for a plain
    split of the rows, the number of sequences for a [B, S, .] activation sharded on S)."""

    def __init__(self, arena: symm.SymmetricArena, ranks: Sequence[int]):
        self.arena, self.ranks = arena, list(ranks)
        self.g = len(self.ranks)
        self.me = self.ranks.index(arena.rank)
        self.sets: Dict[Tuple[int, int], _ScatterBufferSet] = {}
        self.lib = _lib.load()
        self.calls = 0

    def supported(self, M: int, N: int, Kd: int, outer: int, dtype: torch.dtype) -> bool:
        if dtype != torch.bfloat16 or N % 32 or Kd % 8 or outer < 1 or M % (self.g * outer):
            return False
        return (M // (self.g * outer)) % BM == 0

    def _sender_slot(self, sender: int, owner: int) -> int:
        """Index of rank position ``sender`` among the senders of ``owner``."""
        return sender if sender < owner else sender - 1

    def __call__(self, a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, outer: int = 1
                 ) -> torch.Tensor:
        M, Kd = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
        N = b.shape[1] if b_mn else b.shape[0]
        g, me = self.g, self.me
        Ms = M // g
        chunk_rows = M // (g * outer)
        bs = self.sets.get((Ms, N))
        if bs is None:
            bs = self.sets[(Ms, N)] = _ScatterBufferSet(self.arena, Ms, N, g)
        bs.epoch += 1
        par = bs.epoch & 1
        if bs.args[par] is None:
            recv, flags = bs.recv[par], bs.flags[par]
            slot_bytes, flag_bytes = Ms * N * 2, bs.tiles * 4
            my_rank = self.arena.rank
            bs.args[par] = (
                (c_int64 * (g - 1))(*[recv.ptr(my_rank) + p * slot_bytes for p in range(g - 1)]),
                (c_int64 * g)(*[0 if r == me else recv.ptr(self.ranks[r]) + self._sender_slot(me, r) * slot_bytes
                                for r in range(g)]),
                (c_int64 * (g - 1))(*[flags.ptr(my_rank) + p * flag_bytes for p in range(g - 1)]),
                (c_int64 * g)(*[0 if r == me else flags.ptr(self.ranks[r]) + self._sender_slot(me, r) * flag_bytes
                                for r in range(g)]))
        recv_local, recv_peer, flag_local, flag_peer = bs.args[par]
        out = torch.empty((Ms, N), dtype=torch.bfloat16, device=a.device)
        rc = self.lib.mm_gemm_reducescatter_bf16(a.data_ptr(), int(a_mn), a.stride(0), b.data_ptr(), int(b_mn), b.stride(0),
                                                 out.data_ptr(), out.stride(0), M, N, Kd, recv_local, recv_peer,
                                                 flag_local, flag_peer, g, me, chunk_rows, bs.epoch,
                                                 torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "mm_gemm_reducescatter_bf16")
        K._count()
        self.calls += 1
        return out


_lib.register("mm_allgather_gemm_bf16", c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64,
                                                c_void_p, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                                c_void_p])


class FusedAllGatherLinear:
    """``concat_r(A_r) @ B^T`` for row-sharded (sequence-parallel) activations: the kernel pulls
    the peers' row shards over NVLink while its tensor-core main loop already works on the rows
    that have arrived (``mm_allgather_gemm_bf16``). One instance per tensor-parallel group.

    Every rank copies its shard into a peer-visible tile (double-buffered by call parity) and
    raises its flag at the peers behind the copy; there is no barrier ahead of the kernel: its
    helper warps wait for a peer's flag right before they pull that peer's rows, while the
    tensor cores already work on this rank's own rows (read from the caller's tensor, not from
    the copy). A tile is overwritten two calls later; by then this rank has seen the peers'
    flags of the call in between, which they raise only after their kernel of the earlier call
    has finished reading the tile."""

    def __init__(self, arena: symm.SymmetricArena, ranks: Sequence[int]):
        self.arena, self.ranks = arena, list(ranks)
        self.g = len(self.ranks)
        self.me = self.ranks.index(arena.rank)
        self.flag_off = [arena.alloc_flag() for _ in self.ranks]
        self.epoch = 0
        self.sets: Dict[Tuple[int, int], dict] = {}
        self.lib = _lib.load()
        self.calls = 0
        self.barrier_first = os.environ.get("MM_AG_BARRIER", "0") == "1"
        self._peer_flags = None
        self._shard_ready = None

    def _barrier(self) -> None:
        self.epoch += 1
        a = self.arena
        peers = [r for r in self.ranks if r != a.rank]
        symm.set_flags(a, [a.flag_ptr(r, self.flag_off[self.me]) for r in peers], self.epoch)
        symm.wait_flags(a, [a.flag_ptr(a.rank, self.flag_off[self.ranks.index(r)]) for r in peers], self.epoch)

    @staticmethod
    def supported(rows_per_rank: int, Kd: int, outer: int = 1, dtype: torch.dtype = torch.bfloat16) -> bool:
        """``outer`` chunks per rank (1: the shards concatenate; the number of sequences for a
        [B, S, .] activation sharded on S); a chunk must be a whole number of 128-row blocks."""
        return (dtype == torch.bfloat16 and outer >= 1 and rows_per_rank % outer == 0
                and (rows_per_rank // outer) % BM == 0 and Kd % 8 == 0)

    def __call__(self, a_shard: torch.Tensor, b: torch.Tensor, *, b_mn: bool = False, outer: int = 1):
        """Returns ``(C [M, N], A_full [M, K])``; ``A_full`` is the gathered input (kept for the
        weight gradient)."""
        Ms, Kd = a_shard.shape
        M = Ms * self.g
        N = b.shape[1] if b_mn else b.shape[0]
        st = self.sets.get((Ms, Kd))
        if st is None:
            st = self.sets[(Ms, Kd)] = {
                "stage": [self.arena.alloc((Ms, Kd), torch.bfloat16) for _ in range(2)],
                "ready": torch.zeros(M // BM, dtype=torch.int32, device=a_shard.device), "calls": 0,
                "target": c_int(0), "srcs": [None, None]}
        st["calls"] += 1
        par = st["calls"] & 1
        stage = st["stage"][par]
        a_shard = a_shard.contiguous()
        a = self.arena
        stage.peer(a.rank).copy_(a_shard)
        gathered = torch.empty((M, Kd), dtype=torch.bfloat16, device=a_shard.device)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a_shard.device)
        if st["srcs"][par] is None:
            st["srcs"][par] = (c_int64 * self.g)(*[stage.ptr(r) for r in self.ranks])
        srcs = st["srcs"][par]
        if self.barrier_first:       # MM_AG_BARRIER=1: a flag barrier of the group ahead of the kernel (for comparisons)
            self._barrier()
            shard_ready = None
        else:
            self.epoch += 1
            if self._peer_flags is None:
                self._peer_flags = [a.flag_ptr(r, self.flag_off[self.me]) for r in self.ranks if r != a.rank]
                self._shard_ready = (c_int64 * self.g)(*[a.flag_ptr(a.rank, self.flag_off[j]) for j in range(self.g)])
            symm.set_flags(a, self._peer_flags, self.epoch)
            shard_ready = self._shard_ready
        rc = self.lib.mm_allgather_gemm_bf16(srcs, self.g, self.me, gathered.data_ptr(), st["ready"].data_ptr(), ctypes.byref(st["target"]),
                                             b.data_ptr(), int(b_mn), b.stride(0), out.data_ptr(), out.stride(0), M, N, Kd,
                                             Ms // outer, shard_ready, self.epoch, a_shard.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "mm_allgather_gemm_bf16")
        K._count()
        self.calls += 1
        return out, gathered
