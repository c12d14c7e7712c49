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
