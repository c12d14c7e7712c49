"""Cross-submesh reshard execution.

The native planner (``_mm_C.plan_reshard``) intersects source and destination
tiles and yields rectangular chunks ``(src_device, dst_device, box, offsets)``.
Three executors move them:

* ``run_reshard_local``  - all devices live in this process (virtual CPU devices or
  several CUDA devices): the destination pulls every chunk with a strided copy.
* ``run_reshard_dist``   - one process per device without peer-mapped memory
  (CPU/gloo ranks, or the NCCL baseline): chunks travel as point-to-point messages.
* ``p2p_reshard`` (see :mod:`multimesh_jax_b200.parallel.symm`) - the hand-written pull
  kernel that reads source tiles straight from peer HBM.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..compiler.capture import DTYPE_FROM_NAME


def _slices(offset, lo, hi):
    return tuple(slice(o, o + (b - a)) for o, a, b in zip(offset, lo, hi))


def run_reshard_local(topo, device: int, src_tiles: Dict[int, torch.Tensor], chunks: List[dict], dst_shape: dict
                      ) -> torch.Tensor:
    dev = topo.torch_device(device)
    out = torch.empty(dst_shape["shard_size"], dtype=DTYPE_FROM_NAME[dst_shape["dtype"]], device=dev)
    if len(chunks) == 1:
        c = chunks[0]
        src = src_tiles[c["src_device"]]
        piece = src[_slices(c["src_offset"], c["lo"], c["hi"])]
        if list(piece.shape) == list(out.shape):
            # whole tile from one source: a plain (possibly cross-device) copy
            return piece.to(dev, copy=True) if piece.device != dev or not piece.is_contiguous() else piece.clone()
    for c in chunks:
        src = src_tiles[c["src_device"]]
        out[_slices(c["dst_offset"], c["lo"], c["hi"])].copy_(src[_slices(c["src_offset"], c["lo"], c["hi"])])
    return out


class CommStream:
    """Side stream for point-to-point messages of one process (one GPU).

    Messages are issued on this stream, behind everything the compute stream has queued so
    far, so a receive that is posted early does not hold back later compute kernels and a send
    does not wait in front of them. ``run_reshard_dist`` returns an event; the first task that
    reads the received tile makes the compute stream wait for it. Tensors of messages in
    flight are kept referenced here until their event has fired, so the caching allocator
    cannot hand their memory to another stream's kernels."""

    def __init__(self, device: torch.device):
        self.device = device
        self.stream = torch.cuda.Stream(device=device)
        self.pending: List[tuple] = []

    def reap(self) -> None:
        self.pending = [(ev, keep) for ev, keep in self.pending if not ev.query()]

    def drain(self) -> None:
        """Makes the compute stream wait for every message still in flight."""
        cur = torch.cuda.current_stream(self.device)
        for ev, _ in self.pending:
            cur.wait_event(ev)
        self.reap()


def run_reshard_dist(topo, device: int, src_tile: Optional[torch.Tensor], send_chunks: List[dict],
                     recv_chunks: List[dict], dst_shape: dict, comm: Optional[CommStream] = None):
    """Point-to-point realisation: every chunk whose source and destination
    differ is one message; all ranks issue their sends and receives as one batch.
    Returns ``(tile or None, event or None)``: with a :class:`CommStream` the messages run
    on the side stream and the event marks their completion; without one the call returns
    after making the current stream wait for them."""
    import torch.distributed as dist
    dev = topo.torch_device(device)
    out = None
    if recv_chunks:
        out = torch.empty(dst_shape["shard_size"], dtype=DTYPE_FROM_NAME[dst_shape["dtype"]], device=dev)
    ops = []
    staged = []
    keep: List[torch.Tensor] = []
    for c in send_chunks:
        if c["dst_device"] == device:
            continue
        piece = src_tile[_slices(c["src_offset"], c["lo"], c["hi"])].contiguous()
        keep.append(piece)
        ops.append(dist.P2POp(dist.isend, piece, c["dst_device"]))
    for c in recv_chunks:
        view = out[_slices(c["dst_offset"], c["lo"], c["hi"])]
        if c["src_device"] == device:
            view.copy_(src_tile[_slices(c["src_offset"], c["lo"], c["hi"])])
            continue
        if view.is_contiguous():
            ops.append(dist.P2POp(dist.irecv, view, c["src_device"]))
        else:
            tmp = torch.empty(view.shape, dtype=out.dtype, device=dev)
            staged.append((view, tmp))
            keep.append(tmp)
            ops.append(dist.P2POp(dist.irecv, tmp, c["src_device"]))
    if not ops:
        return out, None
    if comm is None:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        for view, tmp in staged:
            view.copy_(tmp)
        return out, None
    comm.reap()
    comm.stream.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(comm.stream):
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        for view, tmp in staged:
            view.copy_(tmp)
        ev = torch.cuda.Event()
        ev.record(comm.stream)
    if out is not None:
        keep.append(out)
    comm.pending.append((ev, keep))
    return out, ev


class PeerReshard:
    """Cross-submesh reshards of a one-process-per-GPU job through peer-mapped memory.

    Every distinct (source buffer, destination buffer) pair of the plan owns two source tiles
    in the symmetric arena (alternating by use) plus ready / done flags. The task that produces
    the source store writes its output straight into the tile of the coming use
    (:meth:`claim_source`: the store's tile *is* the arena tile, nothing is copied); a source
    rank then only raises the ready flags of the ranks that read from it. A destination rank
    waits for its sources' flags and runs the pull kernel, which reads the source tiles
    straight from peer HBM over NVLink and writes the destination layout in one pass (no NCCL
    call, no intermediate receive buffer), then raises the done flags that let the sources
    reuse the tile two uses later. Producers that cannot write into a given tile (interpreted
    task bodies, parameters, a source buffer read by several reshards) have their tile copied
    into the arena first. Waits are bounded by wall-clock time and report through the status
    word. The reference moves cross-submesh data with one call into its task runtime
    (src/pjrt_client/zuku_execute_context_impl.cc:437-452)."""

    MIN_BYTES = 64 << 10

    def __init__(self, arena, topo, plan: dict, buffer_of: Dict[int, int], reshard_plan_of):
        from . import symm
        self.arena, self.topo, self.symm = arena, topo, symm
        self.slots: Dict[tuple, dict] = {}
        self.bytes = 0
        # every pull of this object runs on the side stream, one after the other: one counter word
        self.counter = arena.alloc_counter("PeerReshard")
        self.direct_uses = 0          # uses whose producer wrote into the arena tile itself
        self.copied_uses = 0          # uses that needed the copy into the arena
        for op in plan["ops"]:
            if op["kind"] != "reshard":
                continue
            key = (buffer_of[op["src_store"]], buffer_of[op["dst_store"]])
            if key in self.slots:
                continue
            src, dst = plan["stores"][op["src_store"]]["shape"], plan["stores"][op["dst_store"]]["shape"]
            rplan = reshard_plan_of(op["src_store"], op["dst_store"])
            if not self.pullable(rplan, src, dst):
                self.slots[key] = None
                continue
            dtype = DTYPE_FROM_NAME[src["dtype"]]
            srcs = list(range(src["device_start"], src["device_start"] + src["num_devices"]))
            dsts = list(range(dst["device_start"], dst["device_start"] + dst["num_devices"]))
            readers: Dict[int, List[int]] = {}
            for c in rplan["chunks"]:
                readers.setdefault(c["src_device"], set()).add(c["dst_device"])
            slot = {"stage": [arena.alloc(src["shard_size"], dtype) for _ in range(2)],
                    "ready": [[arena.alloc_flag() for _ in srcs] for _ in range(2)],
                    "done": [[arena.alloc_flag() for _ in dsts] for _ in range(2)],
                    "srcs": srcs, "dsts": dsts, "uses": 0, "claimed": {},
                    "readers": {d: sorted(r) for d, r in readers.items()}}
            self.slots[key] = slot
            n = 1
            for s in src["shard_size"]:
                n *= s
            self.bytes += 2 * n * dtype.itemsize

    def claim_source(self, key, d: int) -> torch.Tensor:
        """The arena tile that the coming use of ``key`` will read on device ``d``, for the
        producer to write its output into. Queues, on the current stream, the wait for the
        readers of the use two back (the last ones to read this tile)."""
        slot = self.slots[key]
        e = slot["uses"] + 1
        par = e & 1
        if slot["claimed"].get(d) != e:
            readers = slot["readers"].get(d, ())
            if e > 2 and readers:
                self.symm.wait_flags(self.arena, [self.arena.flag_ptr(d, slot["done"][par][slot["dsts"].index(r)])
                                                  for r in readers], e - 2)
            slot["claimed"][d] = e
        return slot["stage"][par].peer(d)

    @classmethod
    def required_bytes(cls, plan: dict, buffer_of: Dict[int, int]) -> int:
        """Upper bound of the arena space the staging tiles of ``plan`` need."""
        seen, total = set(), 0
        for op in plan["ops"]:
            if op["kind"] != "reshard":
                continue
            key = (buffer_of[op["src_store"]], buffer_of[op["dst_store"]])
            if key in seen:
                continue
            seen.add(key)
            src = plan["stores"][op["src_store"]]["shape"]
            n = DTYPE_FROM_NAME[src["dtype"]].itemsize
            for s in src["shard_size"]:
                n *= s
            total += 2 * ((n + 1023) // 1024 * 1024)
        return total

    @classmethod
    def pullable(cls, rplan: dict, src: dict, dst: dict) -> bool:
        """Tiles the pull kernel can move: 16-byte aligned rows, at most four dimensions that
        do not merge, and large enough for a kernel of its own to pay off."""
        esz = DTYPE_FROM_NAME[src["dtype"]].itemsize
        sshape, dshape = list(src["shard_size"]), list(dst["shard_size"])
        if not sshape or not rplan["chunks"]:
            return False
        n = esz
        for s in sshape:
            n *= s
        if n < cls.MIN_BYTES or (sshape[-1] * esz) % 16 or (dshape[-1] * esz) % 16:
            return False
        from .symm import build_pull_chunks
        try:
            recs = build_pull_chunks(rplan["chunks"], sshape, dshape, lambda d: 0, 0, esz)
        except NotImplementedError:
            return False
        for r in recs:
            ext, ss, ds = r[2:6], r[6:10], r[10:14]
            if (r[0] % 16) or (r[1] % 16) or (ext[3] * esz) % 16:
                return False
            for k in range(3):
                if ext[k] > 1 and ((ss[k] * esz) % 16 or (ds[k] * esz) % 16):
                    return False
        return True

    def run(self, key, d: int, src_tile: Optional[torch.Tensor], chunks: List[dict], src: dict, dst: dict,
            comm: Optional[CommStream]):
        """This rank's part of one use of ``key``. With a :class:`CommStream` the work is queued
        on that side stream and ``(destination tile or None, event)`` is returned; with ``None``
        it is queued on the current stream (the runtime context chose it and orders the readers
        of the tile behind it) and the event is ``None``."""
        symm, arena, slot = self.symm, self.arena, self.slots[key]
        slot["uses"] += 1
        e = slot["uses"]
        par = e & 1
        mine_src = [c for c in chunks if c["src_device"] == d]
        mine_dst = [c for c in chunks if c["dst_device"] == d]
        dev = self.topo.torch_device(d)
        esz = DTYPE_FROM_NAME[src["dtype"]].itemsize
        out = None
        if mine_dst:
            out = torch.empty(dst["shard_size"], dtype=DTYPE_FROM_NAME[dst["dtype"]], device=dev)
        if comm is None:
            import contextlib
            scope = contextlib.nullcontext()
        else:
            comm.reap()
            comm.stream.wait_stream(torch.cuda.current_stream(dev))
            scope = torch.cuda.stream(comm.stream)
        with scope:
            if mine_src:
                readers = sorted({c["dst_device"] for c in mine_src})
                mine = slot["stage"][par].peer(d)
                if slot["claimed"].get(d) == e and src_tile.data_ptr() == mine.data_ptr():
                    self.direct_uses += 1       # the producer wrote into the arena tile: nothing to move
                else:
                    if e > 2:   # the tile of this parity was last read in use e - 2
                        symm.wait_flags(arena, [arena.flag_ptr(d, slot["done"][par][slot["dsts"].index(r)])
                                                for r in readers], e - 2)
                    mine.copy_(src_tile.view(mine.shape))
                    self.copied_uses += 1
                symm.set_flags(arena, [arena.flag_ptr(r, slot["ready"][par][slot["srcs"].index(d)]) for r in readers], e)
            if mine_dst:
                writers = sorted({c["src_device"] for c in mine_dst})
                symm.wait_flags(arena, [arena.flag_ptr(d, slot["ready"][par][slot["srcs"].index(w)]) for w in writers], e)
                recs = symm.build_pull_chunks(mine_dst, list(src["shard_size"]), list(dst["shard_size"]),
                                              lambda dd: slot["stage"][par].ptr(dd), out.data_ptr(), esz)
                done = [arena.flag_ptr(w, slot["done"][par][slot["dsts"].index(d)]) for w in writers]
                for i in range(0, len(recs), 64):
                    last = i + 64 >= len(recs)
                    symm.reshard_pull(recs[i:i + 64], esz, arena, done_flags=done if last else (), done_value=e,
                                       counter=self.counter)
            ev = None
            if comm is not None:
                ev = torch.cuda.Event()
                ev.record(comm.stream)
        if comm is not None:
            comm.pending.append((ev, [t for t in (src_tile, out) if t is not None]))
        return out, ev
