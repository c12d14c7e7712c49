"""Checkpoint / resume that keeps the per-shard array layout.

The reference has no checkpoint code of its own: training scripts built on it save through
the array API of the framework above it, whose on-disk unit is the *shard* of a sharded array
(one file per device tile plus its index in the global array). This module keeps that
layout for :class:`ShardedTensor` pytrees:

```
<dir>/manifest.json            tree structure, per leaf: dtype, global sizes, sharding descriptor,
                               and for every tile its device ordinal, box [lo, hi) and file name
<dir>/<leaf>.<ordinal>.pt      one tile (written by the process that owns the device)
```

Every process writes only the tiles of its own devices, each to a temporary name that is
renamed into place; rank 0 writes the manifest after a barrier over all ranks, so a manifest
on disk means that every tile it names is complete. Loading
into the same layout reads each tile straight into place; loading into a different layout
(other mesh shape, other device count) assembles every destination tile from the boxes that
intersect it, reading only the files it needs.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

import torch
from torch.utils import _pytree as pytree

from ..compiler.capture import DTYPE_FROM_NAME
from ..runtime.collectives import Topology, tile_box
from ..runtime.executable import ShardedTensor

MANIFEST = "manifest.json"
FORMAT_VERSION = 1


def _is_leaf(x):
    return isinstance(x, ShardedTensor)


def _replica_owner(sharding: dict, ordinal: int) -> int:
    """First ordinal that holds the same box as ``ordinal`` (replicas are saved once)."""
    box = tile_box(sharding, ordinal)
    for o in range(ordinal):
        if tile_box(sharding, o) == box:
            return o
    return ordinal


def _atomic_save(tensor: torch.Tensor, path: str) -> None:
    tmp = f"{path}.tmp.{os.getpid()}"
    torch.save(tensor, tmp)
    os.replace(tmp, path)


def _shard_size(sh: dict) -> List[int]:
    """Tile extents of a layout (every tile of a layout has the same shape)."""
    if "shard_size" in sh:
        return list(sh["shard_size"])
    lo, hi = tile_box(sh, 0)
    return [b - a for a, b in zip(lo, hi)]


def save(directory: str, tree: Any, *, step: Optional[int] = None, rank: Optional[int] = None) -> dict:
    """Writes ``tree`` (a pytree of :class:`ShardedTensor`, tensors and plain values). Returns
    the manifest. In one-process-per-device jobs every rank must call this."""
    os.makedirs(directory, exist_ok=True)
    leaves, spec = pytree.tree_flatten(tree, is_leaf=_is_leaf)
    import torch.distributed as dist
    distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    if rank is None:
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    entries: List[dict] = []
    for i, leaf in enumerate(leaves):
        name = f"leaf{i:05d}"
        if isinstance(leaf, ShardedTensor):
            sh = leaf.sharding
            start = sh["device_start"]
            tiles = []
            local = leaf.local_tiles()
            for o in range(sh["num_devices"]):
                lo, hi = tile_box(sh, o)
                owner = _replica_owner(sh, o)
                fname = f"{name}.{owner}.pt"
                tiles.append({"ordinal": o, "lo": list(lo), "hi": list(hi), "file": fname})
                if owner == o and (start + o) in local:
                    _atomic_save(local[start + o].detach().cpu(), os.path.join(directory, fname))
            entries.append({"kind": "sharded", "dtype": sh["dtype"], "sizes": list(sh["sizes"]),
                            "sharding": dict({k: sh[k] for k in ("dim_axes", "mesh_dims", "device_start", "num_devices",
                                                                 "key")}, shard_size=_shard_size(sh)),
                            "tiles": tiles})
        elif isinstance(leaf, torch.Tensor):
            fname = f"{name}.full.pt"
            if rank == 0:
                _atomic_save(leaf.detach().cpu(), os.path.join(directory, fname))
            entries.append({"kind": "tensor", "file": fname})
        else:
            entries.append({"kind": "value", "value": leaf})
    manifest = {"format": FORMAT_VERSION, "step": step, "treespec": pytree.treespec_dumps(spec), "leaves": entries}
    if distributed:
        dist.barrier()      # every rank's tiles are in place before the manifest can appear
    if rank == 0:
        tmp = os.path.join(directory, MANIFEST + ".tmp")
        with open(tmp, "w") as f:
            json.dump(manifest, f)
        os.replace(tmp, os.path.join(directory, MANIFEST))   # the manifest appears last and atomically
    if distributed:
        dist.barrier()      # no rank returns (and possibly loads) before the manifest exists
    return manifest


def read_manifest(directory: str) -> dict:
    with open(os.path.join(directory, MANIFEST)) as f:
        m = json.load(f)
    if m.get("format") != FORMAT_VERSION:
        raise ValueError(f"unsupported checkpoint format {m.get('format')}")
    return m


def _load_tile(directory: str, entry: dict, lo, hi, cache: Dict[str, torch.Tensor], dtype, device) -> torch.Tensor:
    """Assembles the box [lo, hi) of a saved sharded leaf from the tiles that intersect it."""
    out = torch.empty([b - a for a, b in zip(lo, hi)], dtype=dtype, device=device)
    seen = set()
    for t in entry["tiles"]:
        if t["file"] in seen:
            continue
        ilo = [max(a, c) for a, c in zip(lo, t["lo"])]
        ihi = [min(b, d) for b, d in zip(hi, t["hi"])]
        if any(a >= b for a, b in zip(ilo, ihi)) and len(lo) > 0:
            continue
        seen.add(t["file"])
        if t["file"] not in cache:
            cache[t["file"]] = torch.load(os.path.join(directory, t["file"]), map_location="cpu")
        src = cache[t["file"]]
        s_idx = tuple(slice(a - c, b - c) for a, b, c in zip(ilo, ihi, t["lo"]))
        d_idx = tuple(slice(a - c, b - c) for a, b, c in zip(ilo, ihi, lo))
        out[d_idx] = src[s_idx].to(device)
    return out


def load(directory: str, *, like: Any = None, shardings: Optional[List[Optional[dict]]] = None,
         topology: Optional[Topology] = None) -> Any:
    """Reads a checkpoint. Layout of the result, per sharded leaf:

    * ``like`` given (a pytree with :class:`ShardedTensor` leaves, e.g. the freshly initialised
      state of a newly compiled step): that leaf's sharding and topology - this is how a run is
      resumed on a different mesh;
    * else ``shardings[i]`` if given; else the layout stored in the manifest (needs ``topology``).
    Only tiles of local devices are read."""
    m = read_manifest(directory)
    spec = pytree.treespec_loads(m["treespec"])
    like_leaves = pytree.tree_flatten(like, is_leaf=_is_leaf)[0] if like is not None else None
    if like_leaves is not None and len(like_leaves) != len(m["leaves"]):
        raise ValueError("`like` does not have the structure of the checkpoint")
    out = []
    for i, e in enumerate(m["leaves"]):
        if e["kind"] == "value":
            out.append(e["value"])
            continue
        if e["kind"] == "tensor":
            out.append(torch.load(os.path.join(directory, e["file"]), map_location="cpu"))
            continue
        if like_leaves is not None and isinstance(like_leaves[i], ShardedTensor):
            sh, topo = like_leaves[i].sharding, like_leaves[i].topology
        else:
            sh = (shardings[i] if shardings is not None and shardings[i] is not None else None)
            topo = topology
            if sh is None:
                sh = dict(e["sharding"], dtype=e["dtype"], sizes=e["sizes"])
                sh.setdefault("shard_size", _shard_size(sh))   # manifests written before the field existed
            if topo is None:
                raise ValueError("load() needs `like` or `topology` to place sharded leaves")
        if list(sh["sizes"]) != list(e["sizes"]):
            raise ValueError(f"leaf {i}: checkpoint has shape {e['sizes']}, target layout {sh['sizes']}")
        dtype = DTYPE_FROM_NAME[e["dtype"]]
        cache: Dict[str, torch.Tensor] = {}
        tiles = {}
        for o in range(sh["num_devices"]):
            d = sh["device_start"] + o
            if not topo.is_local(d):
                continue
            lo, hi = tile_box(sh, o)
            tiles[d] = _load_tile(directory, e, lo, hi, cache, dtype, topo.torch_device(d))
        out.append(ShardedTensor(sh, tiles, topo))
    return pytree.tree_unflatten(out, spec)
