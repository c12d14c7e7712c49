"""Process-wide and trace-time state of the front end.

Three tiers of configuration mirror the reference (``jax_plugins/multimesh/init.py:12-34``,
``multimesh/jax/lib.py:50-132``, ``src/pjrt_client/mpmd_utils.cc:42-65``):
``init()`` keyword arguments, Python context managers / setters, and ``MULTIMESH_*``
environment variables read by the C++ passes.
"""
from __future__ import annotations

import contextlib
import os
import threading
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class StartupConfig:
    """Mirror of the options ``init()`` forwards to the native runtime."""
    cpus: int = 0
    gpus: int = 0
    fbmem: int = 8000
    sysmem: int = 4000
    zcmem: int = 32
    network: str = "none"
    kthreads: int = 0
    profile: bool = False
    debug: int = 0
    dump: Optional[str] = None
    dump_all_passes: bool = False
    argv: List[str] = field(default_factory=list)
    distributed: bool = False
    initialized: bool = False


class _Flags(threading.local):
    def __init__(self):
        self.autoshard = False
        self.ignore_transforms = False
        self.fast_path = True
        self.recomputation = True
        self.metadata_name_tasks = True


@dataclass
class ScopeEntry:
    """One entry of the trace-time name stack."""
    name: str
    explicit_task: Optional[Dict[str, Any]] = None  # payload of an explicit task()


class TraceState:
    """State that exists only while a step function is being captured. It is process-wide
    on purpose: the autograd engine runs the backward pass of CUDA tensors on its own
    worker threads, and the nodes created there must see the same tables."""

    def __init__(self):
        self.active = False
        self.scopes: List[ScopeEntry] = []
        self.loop: Optional[Dict[str, Any]] = None      # config of the microbatch loop being traced
        self.loop_configs: List[Dict[str, Any]] = []     # every loop seen in this capture
        self.scope_by_seq: Dict[int, Any] = {}           # autograd sequence nr -> node tag
        self.task_counter = 0

    def reset(self):
        self.__init__()

    def current_tag(self):
        names = [s.name for s in self.scopes if s.name]
        explicit = None
        for s in reversed(self.scopes):
            if s.explicit_task is not None:
                explicit = s.explicit_task
                break
        return {"scope": "/".join(names), "task": explicit,
                "loop": self.loop["id"] if self.loop else -1}


startup = StartupConfig()
flags = _Flags()
trace = TraceState()

# Global knobs that map to C++ globals in the reference
# (``src/pjrt_client/mm_pjrt_client.cc:51-54``).
knobs = {
    "replicated_parameter_num_elements_cutoff": 0,
    "recompute_from_arguments_if_cost_less_than": 1 << 20,
    # open a named profiler / NVTX range around every task launch (MM_TASK_RANGES=1, or set by
    # utils.timeline.profile); off by default because it costs a few microseconds per task
    "task_ranges": os.environ.get("MM_TASK_RANGES", "0") == "1",
}


@contextlib.contextmanager
def _flag(name: str, value):
    old = getattr(flags, name)
    setattr(flags, name, value)
    try:
        yield
    finally:
        setattr(flags, name, old)
