"""multimesh_jax_b200: a Blackwell-native MPMD parallelism runtime for PyTorch.

The public names follow the reference package (``multimesh/jax/__init__.py:4-39``).
"""
from __future__ import annotations

import importlib
import os as _os


def _load_native():
    """Imports the native compiler/runtime module, building it in-tree on first use."""
    try:
        return importlib.import_module(__name__ + "._mm_C")
    except ImportError:
        from .csrc.build import build_host
        build_host()
        importlib.invalidate_caches()
        return importlib.import_module(__name__ + "._mm_C")


_mm_C = _load_native()

from . import state  # noqa: E402
from .lib import (autoshard, context, custom_partitioning, enable_fast_path, enable_recomputation,  # noqa: E402
                  ignore_transforms, index_class, mjit, optional_kwargs, shard_map,
                  recompute_from_arguments_if_cost_less_than, relayout, replicate_parameters_smaller_than_num_elements,
                  should_ignore_transforms, tasks, with_sharding_constraint)
from .no_op import mark_gradient, mark_loss, no_op  # noqa: E402
from .task import (Context, MultiMesh, Task, TaskMesh, clear_tasks, microbatch, module_scopes, named_scope,  # noqa: E402
                   parallelize, register_task, get_abstract_global_mesh, get_global_mesh, slice_global_mesh, task,
                   value_and_grad)
from .runtime.executable import Executable, ShardedTensor, StepFailed  # noqa: E402
from .compiler.api import compile_function, compile_program_file  # noqa: E402
from .init import detect_cluster, init, init_test, shutdown  # noqa: E402

__all__ = [
    "task", "microbatch", "parallelize", "register_task", "slice_global_mesh", "Task", "TaskMesh", "Context",
    "MultiMesh", "autoshard", "context", "enable_fast_path", "enable_recomputation", "ignore_transforms",
    "with_sharding_constraint", "relayout", "tasks", "mjit", "shutdown", "replicate_parameters_smaller_than_num_elements",
    "recompute_from_arguments_if_cost_less_than", "clear_tasks", "no_op", "mark_gradient", "mark_loss",
    "value_and_grad", "named_scope", "module_scopes", "compile_function", "compile_program_file", "Executable", "ShardedTensor",
    "StepFailed", "init", "init_test", "custom_partitioning", "index_class", "shard_map", "detect_cluster",
    "get_global_mesh", "get_abstract_global_mesh", "optional_kwargs",
]
