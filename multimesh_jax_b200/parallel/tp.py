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
from ctypes import c_int, c_int64, c_void_p
from typing import Dict, List, Sequence, Tuple

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
