"""Peer-mapped symmetric memory for one-process-per-GPU jobs.

Every rank allocates an arena with ``cudaMalloc`` (outside PyTorch's caching
allocator, so that it can be exported), shares it through CUDA IPC handles
exchanged over ``torch.distributed`` and maps the arenas of all other ranks of
the node. Tensors carved out of the arena at the *same offset on every rank*
are "symmetric": a kernel on rank ``r`` can address the copy of rank ``p`` as
``peer_base[p] + offset`` - plain loads and stores over NVLink, issued from
inside our kernels (never TMA multicast).

The first ``FLAG_BYTES`` of each arena hold epoch counters used as ready /
consumed flags by the fused kernels; every wait on them is bounded.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int64, c_size_t, c_void_p
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import _lib
from ..ops import kernels as K

FLAG_BYTES = 1 << 16
_ALIGN = 1024

_lib.register("mm_peer_alloc", c_int, [ctypes.POINTER(c_void_p), c_size_t])
_lib.register("mm_peer_free", c_int, [c_void_p])
_lib.register("mm_ipc_get_handle", c_int, [c_void_p, c_void_p])
_lib.register("mm_ipc_open_handle", c_int, [c_void_p, ctypes.POINTER(c_void_p)])
_lib.register("mm_ipc_close", c_int, [c_void_p])
_lib.register("mm_enable_peer_access", c_int, [c_int])
_lib.register("mm_reshard_pull", c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                         c_void_p, c_int, c_void_p])
_lib.register("mm_set_flag", c_int, [c_void_p, c_int, c_void_p])
_lib.register("mm_wait_flag", c_int, [c_void_p, c_int, c_void_p])
_lib.register("mm_set_flags", c_int, [c_void_p, c_int, c_int, c_void_p])
_lib.register("mm_wait_flags", c_int, [c_void_p, c_int, c_int, c_int, c_void_p])


class WordAllocator:
    """Bookkeeping of the 4-byte words at the start of an arena: the first ``NUM_COUNTERS`` are
    CTA counters (one per launcher, handed out once, never shared), the rest are flags."""

    NUM_COUNTERS = 64

    def __init__(self, total_words: int):
        self.total_words = total_words
        self.counter_owner: Dict[int, str] = {}
        self._next_flag = self.NUM_COUNTERS

    def alloc_counter(self, owner: str) -> int:
        index = len(self.counter_owner)
        if index >= self.NUM_COUNTERS:
            raise MemoryError("all CTA-counter words of the arena are taken")
        self.counter_owner[index] = owner
        return index

    def alloc_flag(self) -> int:
        off = self._next_flag * 4
        self._next_flag += 1
        if self._next_flag > self.total_words:
            raise MemoryError("flag area exhausted")
        return off


class _RawCudaBuffer:
    """Exposes a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def tensor_from_ptr(ptr: int, shape: Sequence[int], dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= s
    raw = torch.as_tensor(_RawCudaBuffer(ptr, n * dtype.itemsize), device=device)
    return raw.view(dtype).view(*shape)


class SymmetricArena:
    """One arena per rank, mapped by all ranks of ``group_ranks`` (default: everyone)."""

    def __init__(self, nbytes: int, device: torch.device, ranks: Optional[Sequence[int]] = None):
        import torch.distributed as dist
        self.device = device
        self.lib = _lib.load()
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.ranks = list(ranks) if ranks is not None else list(range(self.world))
        self.nbytes = (nbytes + FLAG_BYTES + _ALIGN - 1) // _ALIGN * _ALIGN
        base = c_void_p()
        _lib.check(self.lib.mm_peer_alloc(ctypes.byref(base), self.nbytes), "mm_peer_alloc")
        self.base = base.value
        handle = ctypes.create_string_buffer(64)
        _lib.check(self.lib.mm_ipc_get_handle(self.base, handle), "mm_ipc_get_handle")
        self.peer_base: Dict[int, int] = {self.rank: self.base}
        self._opened: List[int] = []
        if self.world > 1:
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, handle.raw)
            for r in self.ranks:
                if r == self.rank:
                    continue
                out = c_void_p()
                buf = ctypes.create_string_buffer(handles[r], 64)
                _lib.check(self.lib.mm_ipc_open_handle(buf, ctypes.byref(out)), "mm_ipc_open_handle")
                self.peer_base[r] = out.value
                self._opened.append(out.value)
        self._offset = FLAG_BYTES
        self._named: Dict[str, Tuple[int, int]] = {}
        self.words = WordAllocator(FLAG_BYTES // 4)
        self.epoch = 0

    # -- allocation (must be called in the same order with the same sizes on every rank) ----
    def alloc(self, shape: Sequence[int], dtype: torch.dtype, name: Optional[str] = None) -> "SymmetricTensor":
        n = 1
        for s in shape:
            n *= s
        nbytes = (n * dtype.itemsize + _ALIGN - 1) // _ALIGN * _ALIGN
        if name is not None and name in self._named:
            off, size = self._named[name]
            if size < nbytes:
                raise RuntimeError(f"symmetric buffer {name!r} was created smaller than requested")
        else:
            off = self._offset
            if off + nbytes > self.nbytes:
                raise MemoryError(f"symmetric arena exhausted ({self.nbytes} bytes)")
            self._offset += nbytes
            if name is not None:
                self._named[name] = (off, nbytes)
        return SymmetricTensor(self, off, tuple(shape), dtype)

    def reset(self) -> None:
        self._offset = FLAG_BYTES
        self._named.clear()

    def alloc_flag(self) -> int:
        """Offset (bytes) of a fresh 4-byte flag in the flag area."""
        return self.words.alloc_flag()

    def flag_ptr(self, rank: int, offset: int) -> int:
        return self.peer_base[rank] + offset

    def alloc_counter(self, owner: str) -> int:
        """Index of a zero-initialised CTA-counter word that belongs to ``owner`` alone. A pull
        kernel counts its finished CTAs in the word it is given; two launchers whose kernels can
        overlap on the GPU (different streams) must therefore never share one."""
        return self.words.alloc_counter(owner)

    def counter_ptr(self, index: int) -> int:
        return self.base + 4 * index

    def barrier(self) -> None:
        """Host-side rendezvous: all prior work of every rank has finished."""
        import torch.distributed as dist
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier()

    def close(self) -> None:
        for p in self._opened:
            self.lib.mm_ipc_close(p)
        self._opened.clear()
        if self.base:
            self.lib.mm_peer_free(self.base)
            self.base = 0


class SymmetricTensor:
    """A tensor that exists at the same arena offset on every rank."""

    def __init__(self, arena: SymmetricArena, offset: int, shape: Tuple[int, ...], dtype: torch.dtype):
        self.arena = arena
        self.offset = offset
        self.shape = shape
        self.dtype = dtype
        self.local = tensor_from_ptr(arena.base + offset, shape, dtype, arena.device)

    def ptr(self, rank: int) -> int:
        return self.arena.peer_base[rank] + self.offset

    def peer(self, rank: int) -> torch.Tensor:
        """A tensor view of ``rank``'s copy (peer memory: for our kernels only, never to be
        handed to a library kernel)."""
        return tensor_from_ptr(self.ptr(rank), self.shape, self.dtype, self.arena.device)


_default_arena: Optional[SymmetricArena] = None


def default_arena(nbytes: int = 2 << 30) -> SymmetricArena:
    global _default_arena
    if _default_arena is None:
        dev = torch.device("cuda", torch.cuda.current_device())
        _default_arena = SymmetricArena(nbytes, dev)
    return _default_arena


# ---------------------------------------------------------------------------
# Reshard through the pull kernel
# ---------------------------------------------------------------------------
def _strides(shape: Sequence[int]) -> List[int]:
    st = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        st[i] = st[i + 1] * shape[i + 1]
    return st


def build_pull_chunks(chunks: List[dict], src_tile_shape: Sequence[int], dst_tile_shape: Sequence[int],
                      src_ptr_of_device, dst_ptr: int, elem_size: int) -> List[List[int]]:
    """Turns planner chunks (boxes) into kernel records with at most four dimensions
    (leading dimensions are split into several records when the rank is larger)."""
    records: List[List[int]] = []
    src_shape0, dst_shape0 = list(src_tile_shape), list(dst_tile_shape)
    # The kernel walks the records in order, so at any moment a destination reads mostly from
    # one source. Start every destination at a different source (its own ordinal first, then
    # the next ones in ring order): otherwise all destinations would pull from source 0 first
    # and share that GPU's NVLink egress while the other sources sit idle.
    sources = sorted({c["src_device"] for c in chunks})
    if len(sources) > 1:
        pos = {d: i for i, d in enumerate(sources)}
        chunks = [c for _, c in sorted(enumerate(chunks), key=lambda ic: (
            (pos[ic[1]["src_device"]] - ic[1]["dst_device"]) % len(sources), ic[0]))]
    for c in chunks:
        src_tile_shape, dst_tile_shape = list(src_shape0), list(dst_shape0)   # merged per chunk below
        s_str, d_str = _strides(src_tile_shape), _strides(dst_tile_shape)
        ext = [h - l for l, h in zip(c["lo"], c["hi"])]
        nd = len(ext)
        # merge trailing dimensions that are contiguous in both tiles
        ext2, ss, ds = list(ext), list(s_str), list(d_str)
        so, do = list(c["src_offset"]), list(c["dst_offset"])
        while len(ext2) > 1 and ext2[-1] == src_tile_shape[len(ext2) - 1] == dst_tile_shape[len(ext2) - 1] \
                and so[len(ext2) - 1] == 0 and do[len(ext2) - 1] == 0:
            k = len(ext2) - 1
            ext2[k - 1:] = [ext2[k - 1] * ext2[k]]
            # offsets of dim k-1 are now in units of the merged row
            so[k - 1:] = [so[k - 1] * src_tile_shape[k]]
            do[k - 1:] = [do[k - 1] * dst_tile_shape[k]]
            ss[k - 1:] = [1]
            ds[k - 1:] = [1]
            src_tile_shape = list(src_tile_shape[:k - 1]) + [src_tile_shape[k - 1] * src_tile_shape[k]]
            dst_tile_shape = list(dst_tile_shape[:k - 1]) + [dst_tile_shape[k - 1] * dst_tile_shape[k]]
            s_str, d_str = _strides(src_tile_shape), _strides(dst_tile_shape)
            ss, ds = list(s_str), list(d_str)
        src_base = src_ptr_of_device(c["src_device"]) + sum(o * st for o, st in zip(so, ss)) * elem_size
        dst_base = dst_ptr + sum(o * st for o, st in zip(do, ds)) * elem_size
        if len(ext2) > 4:
            raise NotImplementedError("reshard of tiles with more than four non-mergeable dimensions")
        pad = 4 - len(ext2)
        records.append([src_base, dst_base] + [1] * pad + ext2 + [0] * pad + ss + [0] * pad + ds)
    return records


def reshard_pull(records: List[List[int]], elem_size: int, arena: SymmetricArena, wait_flags: Sequence[int] = (),
                 wait_value: int = 0, done_flags: Sequence[int] = (), done_value: int = 0, max_ctas: int = 0,
                 counter: Optional[int] = None) -> None:
    """Launches the pull kernel on the current stream. ``counter`` is the caller's own CTA-counter
    word (``arena.alloc_counter``); it is needed only with ``done_flags``, which the last CTA to
    finish raises."""
    lib = arena.lib
    if done_flags and counter is None:
        raise ValueError("a pull that raises done flags needs the launcher's own counter word")
    flat = (c_int64 * (14 * len(records)))(*[x for r in records for x in r])
    waits = (c_int64 * max(1, len(wait_flags)))(*wait_flags) if wait_flags else None
    dones = (c_int64 * max(1, len(done_flags)))(*done_flags) if done_flags else None
    rc = lib.mm_reshard_pull(flat, len(records), elem_size, waits, len(wait_flags), wait_value, dones,
                             len(done_flags), done_value, arena.counter_ptr(counter) if done_flags else None, max_ctas,
                             torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "mm_reshard_pull")
    K._count()


def set_flags(arena: SymmetricArena, ptrs: Sequence[int], value: int) -> None:
    """Raises the flags at ``ptrs`` (local or peer addresses) after the stream's earlier work."""
    for i in range(0, len(ptrs), 8):
        part = list(ptrs[i:i + 8])
        arr = (c_int64 * len(part))(*part)
        _lib.check(arena.lib.mm_set_flags(arr, len(part), value, torch.cuda.current_stream().cuda_stream), "mm_set_flags")
        K._count()


def wait_flags(arena: SymmetricArena, ptrs: Sequence[int], value: int, limit_ms: int = 30000) -> None:
    """Holds the current stream until the local flags at ``ptrs`` reach ``value`` (bounded by
    ``limit_ms`` of wall-clock time, after which the device status word records the expiry)."""
    for i in range(0, len(ptrs), 8):
        part = list(ptrs[i:i + 8])
        arr = (c_int64 * len(part))(*part)
        _lib.check(arena.lib.mm_wait_flags(arr, len(part), value, limit_ms, torch.cuda.current_stream().cuda_stream),
                   "mm_wait_flags")
        K._count()
