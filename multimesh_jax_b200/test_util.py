"""Differential test harness: run a function eagerly with every transform ignored (the
reference result) and again MPMD-compiled, compare the results, and check that the compiled
step took its arguments in the layouts that were asked for.

Counterpart of ``multimesh/jax/test_util.py:16-95``. Usable from ``unittest`` (mix
:class:`MultiMeshTestCase` in) or directly through :func:`check_against_reference`.
"""
from __future__ import annotations

import unittest
from typing import Any, Callable, Optional, Sequence

import torch
from torch.utils import _pytree as pytree

from . import lib
from .lib import _canonical_axes
from .runtime.executable import ShardedTensor
from .task import MultiMesh


def _to_global(x):
    return x.full_tensor() if isinstance(x, ShardedTensor) else x


def check_against_reference(f: Callable, arg_maker: Callable[[], Sequence[Any]], *,
                            mesh: Optional[MultiMesh] = None, num_devices: Optional[int] = None,
                            arg_shardings: Optional[Sequence[Any]] = None, donate_argnums: Sequence[int] = (),
                            enable_fast_path: bool = False, backend: Optional[str] = "cpu",
                            atol: Optional[float] = None, rtol: Optional[float] = None):
    """Runs ``f(*arg_maker())`` twice - eagerly under ``ignore_transforms()`` and compiled -
    and asserts that all results agree. ``arg_shardings`` (one entry per argument: ``None`` or
    a tuple of mesh-axis names per dimension) are imposed on the compiled step and verified
    against the layouts the compiler reports. Returns ``(reference, result, executable)``."""
    from .compiler.api import compile_function
    with lib.ignore_transforms():
        ref = f(*arg_maker())
    args = tuple(arg_maker())
    ctx = mesh if mesh is not None else lib.context()
    with lib.enable_fast_path(enable_fast_path), ctx:
        exe = compile_function(f, args, mesh=mesh, num_devices=num_devices, donate_argnums=tuple(donate_argnums),
                               backend=backend, in_shardings=arg_shardings)
        if arg_shardings is not None and hasattr(exe, "input_shardings"):
            got = exe.input_shardings()
            flat_args, _ = pytree.tree_flatten(args)
            flat_specs = []
            for a, spec in zip(args, arg_shardings):
                leaves = pytree.tree_leaves(a)
                flat_specs.extend([spec] * len(leaves))
            tensor_pos = [i for i, a in enumerate(flat_args) if isinstance(a, torch.Tensor)]
            for k, pos in enumerate(tensor_pos):
                spec, sh = flat_specs[pos], got[k]
                if sh is None:
                    continue
                if spec is None:
                    continue   # compiler's choice
                want = _canonical_axes(spec, flat_args[pos].dim())
                names = None
                if mesh is not None and list(sh["mesh_dims"]) == list(mesh.axis_sizes):
                    names = list(mesh.axis_names)
                have = [[names[a] if names else a for a in axes] for axes in sh["dim_axes"]]
                if names and have != want:
                    raise AssertionError(f"argument {pos}: requested layout {want}, compiled layout {have}")
        out = exe(*args)
    ref_leaves = pytree.tree_leaves(ref)
    out_leaves = [_to_global(x) for x in pytree.tree_leaves(out, is_leaf=lambda x: isinstance(x, ShardedTensor))]
    if len(ref_leaves) != len(out_leaves):
        raise AssertionError(f"{len(ref_leaves)} reference results, {len(out_leaves)} compiled results")
    for r, o in zip(ref_leaves, out_leaves):
        if isinstance(r, torch.Tensor):
            torch.testing.assert_close(o.to(r.device), r, atol=atol, rtol=rtol)
        else:
            assert r == o, (r, o)
    return ref, out, exe


class MultiMeshTestCase(unittest.TestCase):
    """``unittest`` flavour of :func:`check_against_reference`."""

    def _test_against_reference(self, f, arg_maker, **kwargs):
        ref, out, exe = check_against_reference(f, arg_maker, **kwargs)
        if hasattr(exe, "shutdown"):
            exe.shutdown()
        return ref, out
