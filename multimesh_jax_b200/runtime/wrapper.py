"""Pass-through executable for programs the MPMD runtime has nothing to do for.

Two kinds of program end up here (``compile_function`` decides):

* the **fast path**: one task, fewer than ``FAST_PATH_MAX_NODES`` operators, no marker operator
  (no ``task``, ``microbatch`` or sharding annotation) - the counterpart of the reference compiling
  such programs with the native client as well and dispatching to that executable
  (``src/pjrt_client/mm_pjrt_client.cc:587-617``, ``src/pjrt_client/mm_pjrt_executable.cc:327-360``);
* the **single-device bypass**: a device assignment of one device and nothing to partition
  (``src/pjrt_client/mm_pjrt_client.cc:525-534``).

``WrapperExecutable`` plays the part of ``WrapperPjRtExecutable``
(``src/pjrt_client/mm_pjrt_executable.cc:45-140``): it unwraps :class:`ShardedTensor` arguments,
runs the captured graph module directly on every local device of the assignment - no task
graph, no stores, no dependence analysis - and wraps the results as replicated
:class:`ShardedTensor` objects so that they can feed a partitioned step without a copy on the
device that computed them.
"""
from __future__ import annotations

from typing import Any, List, Optional

import torch
from torch.utils import _pytree as pytree

from .collectives import Topology
from .executable import ShardedTensor


class WrapperExecutable:
    #: how many times any wrapper ran a step (tests assert that the MPMD runtime was not entered)
    total_calls = 0

    def __init__(self, cap, plan: dict, topology: Topology, *, name: str, reason: str, num_devices: int):
        from .. import _mm_C
        from ..compiler.capture import dtype_name
        self.cap, self.plan, self.topology, self.name = cap, plan, topology, name
        self.reason = reason                 # "fast-path" or "single-device"
        self.num_devices = num_devices
        self.context = None                  # no task-graph runtime behind this executable
        self.launches = 0
        self.calls = 0
        self._out_shardings: List[dict] = []
        g = cap.graph
        for vid in cap.output_values:
            v = g.value(vid)
            self._out_shardings.append(_mm_C.sharded_shape(v["dtype"], list(v["shape"]), [[] for _ in v["shape"]],
                                                           [num_devices], 0))
        self._in_shardings: List[Optional[dict]] = []
        for vid in g.inputs:
            v = g.value(vid)
            self._in_shardings.append(_mm_C.sharded_shape(v["dtype"], list(v["shape"]), [[] for _ in v["shape"]],
                                                          [num_devices], 0))

    # ------------------------------------------------------------------ façade of Executable
    def input_shardings(self) -> List[Optional[dict]]:
        return list(self._in_shardings)

    def output_shardings(self) -> List[dict]:
        return list(self._out_shardings)

    def shard_argument(self, argnum: int, value: Any) -> Any:
        """Argument ``argnum`` (a pytree of global tensors) as replicated :class:`ShardedTensor`
        leaves on the local devices of the assignment."""
        from .executable import shard_tensor
        cap = self.cap
        example = pytree.tree_unflatten(list(range(len(cap.input_is_tensor))), cap.in_spec)
        positions = pytree.tree_leaves(example[argnum])
        tensor_index, k = {}, 0
        for i, ok in enumerate(cap.input_is_tensor):
            if ok:
                tensor_index[i] = k
                k += 1
        leaves, spec = pytree.tree_flatten(value)
        out = []
        for pos, leaf in zip(positions, leaves):
            if pos in tensor_index and isinstance(leaf, torch.Tensor):
                out.append(shard_tensor(leaf, self._in_shardings[tensor_index[pos]], self.topology))
            else:
                out.append(leaf)
        return pytree.tree_unflatten(out, spec)

    def wait(self) -> None:
        for d in self.topology.local_devices:
            dev = self.topology.torch_device(d)
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)

    def event_log(self):
        return []

    def shutdown(self) -> None:
        pass

    # ------------------------------------------------------------------ run
    def __call__(self, *args):
        cap, topo = self.cap, self.topology
        flat, _ = pytree.tree_flatten(tuple(args), is_leaf=lambda x: isinstance(x, ShardedTensor))
        tensors = [a for a in flat if isinstance(a, (torch.Tensor, ShardedTensor))]
        if len(tensors) != cap.num_inputs:
            raise ValueError(f"expected {cap.num_inputs} tensor arguments, got {len(tensors)}")
        self.calls += 1
        WrapperExecutable.total_calls += 1
        per_device: List[List[torch.Tensor]] = []
        locals_ = [d for d in topo.local_devices if d < self.num_devices]
        for d in locals_:
            dev = topo.torch_device(d)
            ins = []
            for a in tensors:
                if isinstance(a, ShardedTensor):
                    tiles = a.local_tiles()
                    replicated = all(len(ax) == 0 for ax in a.sharding["dim_axes"])
                    a = tiles[d] if replicated and d in tiles else a.full_tensor()
                ins.append(a if a.device == dev else a.to(dev))
            if dev.type == "cuda":
                with torch.cuda.device(dev):
                    outs = cap.gm(*ins)
            else:
                outs = cap.gm(*ins)
            per_device.append(list(outs))
            self.launches += 1
        results: List[Any] = []
        it = iter(range(len(cap.output_values)))
        n_out = len(cap.output_values) + len(cap.output_constants)
        for pos in range(n_out):
            if pos in cap.output_constants:
                results.append(cap.output_constants[pos])
                continue
            k = next(it)
            tiles = {d: per_device[i][k] for i, d in enumerate(locals_)}
            results.append(ShardedTensor(self._out_shardings[k], tiles, topo))
        return pytree.tree_unflatten(results, cap.out_spec)
