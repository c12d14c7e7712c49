"""Shard-by-shard initialisation of parameters and optimiser state.

For multi-billion-parameter models the global arrays never exist in one place: every
process creates only the tiles that the compiled step assigns to its devices (the layout
chosen by the compiler is read back from the executable, as ``parallelize`` does in the
reference, ``multimesh/jax/task.py:687-699``)."""
from __future__ import annotations

import math
from typing import Any, Dict, Tuple

import torch
from torch.utils import _pytree as pytree

from ..compiler.capture import DTYPE_FROM_NAME
from ..runtime.collectives import tile_box
from ..runtime.executable import Executable, ShardedTensor
from . import llama


def _tile_like(sharding: dict, topo, fill, generator_seed: int) -> Dict[int, torch.Tensor]:
    tiles = {}
    start = sharding["device_start"]
    for o in range(sharding["num_devices"]):
        d = start + o
        if not topo.is_local(d):
            continue
        dev = topo.torch_device(d)
        shape = sharding["shard_size"]
        dtype = DTYPE_FROM_NAME[sharding["dtype"]]
        # seeded by the tile's position in the array, so replicas of a tile start out identical
        lo, _ = tile_box(sharding, o)
        where = sum((int(x) + 1) * pr for x, pr in zip(lo, (7919, 104723, 1299709, 15485863, 32452843)))
        tiles[d] = fill(shape, dtype, dev, generator_seed + where)
    return tiles


def init_sharded_llama(cfg: llama.LlamaConfig, exe: Executable, device, seed: int = 0) -> Tuple[Any, Any]:
    """Returns ``(params, opt_state)`` as pytrees of :class:`ShardedTensor` laid out the way
    ``exe`` (compiled from ``make_train_step``) expects its first two arguments."""
    topo = exe.topology
    with torch.device("meta"):
        a_params = llama.init_params(cfg, device="meta")
        a_state = llama.init_opt_state(a_params)
    p_leaves, p_spec = pytree.tree_flatten(a_params)
    s_leaves, s_spec = pytree.tree_flatten(a_state)
    shardings = exe.input_shardings()
    n_p = len(p_leaves)
    paths = [pytree.keystr(k) for k, _ in pytree.tree_flatten_with_path(a_params)[0]]
    res_std = 0.02 / math.sqrt(2 * cfg.n_layers)

    def normal(std):
        def fill(shape, dtype, dev, s):
            g = torch.Generator(device=dev).manual_seed(s)
            return (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * std).to(dtype)
        return fill

    def ones(shape, dtype, dev, s):
        return torch.ones(shape, dtype=dtype, device=dev)

    def zeros(shape, dtype, dev, s):
        return torch.zeros(shape, dtype=dtype, device=dev)

    params = []
    for i, (leaf, path) in enumerate(zip(p_leaves, paths)):
        sh = shardings[i]
        if sh is None:
            params.append(torch.zeros(leaf.shape, dtype=leaf.dtype, device=device))
            continue
        if "norm" in path:
            fill = ones
        elif "wo" in path or "wdown" in path:
            fill = normal(res_std)
        else:
            fill = normal(0.02)
        params.append(ShardedTensor(sh, _tile_like(sh, topo, fill, seed + 104729 * i), topo))
    # optimiser state: master = fp32 copy of the working weights, moments = 0, step = 0
    state = []
    for j, leaf in enumerate(s_leaves):
        sh = shardings[n_p + j]
        if sh is None:
            state.append(torch.zeros(leaf.shape, dtype=leaf.dtype, device=device))
            continue
        if j < n_p and isinstance(params[j], ShardedTensor):  # master weights follow the parameter order
            src = params[j]
            if src.sharding["dim_axes"] == sh["dim_axes"] and src.sharding["device_start"] == sh["device_start"]:
                tiles = {d: t.float() for d, t in src.local_tiles().items()}
                state.append(ShardedTensor(sh, tiles, topo))
                continue
        state.append(ShardedTensor(sh, _tile_like(sh, topo, zeros, 0), topo))
    return pytree.tree_unflatten(params, p_spec), pytree.tree_unflatten(state, s_spec)
