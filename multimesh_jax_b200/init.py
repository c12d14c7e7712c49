"""Process start-up: ``init()`` / ``init_test()`` / ``shutdown()``.

Counterpart of ``jax_plugins/multimesh/init.py:12-200``. There is no plugin to
register: ``init`` records the start-up configuration (device counts, memory
budgets, debug level, dump directory), sets the ``MULTIMESH_*`` environment
defaults, and - for ``distributed=True`` - brings up ``torch.distributed``
(NCCL on GPUs, gloo on CPUs), one process per device.
"""
from __future__ import annotations

import argparse
import atexit
import logging
import os
from typing import List, Optional

import torch

from . import state

_log = logging.getLogger("multimesh_jax_b200")


def init(cpus: int = 0, gpus: int = 0, fbmem: int = 8000, sysmem: int = 4000, zcmem: int = 32, debug: int = 0,
         network: str = "none", kthreads: int = 0, profile: bool = False, distributed: bool = False,
         dump: Optional[str] = None, dump_all_passes: bool = False, realm_argv: Optional[List[str]] = None,
         coordinator_address: Optional[str] = None, num_processes: Optional[int] = None,
         process_id: Optional[int] = None, local_device_ids: Optional[List[int]] = None,
         initialization_timeout: int = 300) -> state.StartupConfig:
    cfg = state.startup
    cfg.cpus, cfg.gpus, cfg.fbmem, cfg.sysmem, cfg.zcmem = cpus, gpus, fbmem, sysmem, zcmem
    cfg.network, cfg.kthreads, cfg.profile, cfg.debug = network, kthreads, profile, debug
    cfg.dump, cfg.dump_all_passes, cfg.argv = dump, dump_all_passes, list(realm_argv or [])
    cfg.distributed = distributed
    logging.basicConfig()
    _log.setLevel({0: logging.WARNING, 1: logging.INFO}.get(debug, logging.DEBUG))
    if distributed:
        import datetime
        import torch.distributed as dist
        if not dist.is_initialized():
            if coordinator_address:
                host, _, port = coordinator_address.partition(":")
                os.environ.setdefault("MASTER_ADDR", host or "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", port or "29500")
            if num_processes is not None:
                os.environ.setdefault("WORLD_SIZE", str(num_processes))
            if process_id is not None:
                os.environ.setdefault("RANK", str(process_id))
            use_cuda = torch.cuda.is_available() and gpus != 0
            if use_cuda:
                local = int(os.environ.get("LOCAL_RANK", (local_device_ids or [0])[0]))
                torch.cuda.set_device(local)
            dist.init_process_group("nccl" if use_cuda else "gloo",
                                    timeout=datetime.timedelta(seconds=initialization_timeout))
    cfg.initialized = True
    return cfg


def init_test(argv: Optional[List[str]] = None) -> state.StartupConfig:
    """Command-line mirror of :func:`init` for test programs
    (``--cpus --gpus --network --debug --kthreads --dump --dump-all-passes``)."""
    p = argparse.ArgumentParser(add_help=False)
    p.add_argument("--cpus", type=int, default=0)
    p.add_argument("--gpus", type=int, default=0)
    p.add_argument("--network", default="none")
    p.add_argument("--debug", type=int, default=0)
    p.add_argument("--kthreads", type=int, default=0)
    p.add_argument("--dump", default=None)
    p.add_argument("--dump-all-passes", action="store_true")
    ns, _ = p.parse_known_args(argv)
    return init(cpus=ns.cpus, gpus=ns.gpus, network=ns.network, debug=ns.debug, kthreads=ns.kthreads,
                dump=ns.dump, dump_all_passes=ns.dump_all_passes)


def shutdown() -> None:
    """Drains and stops every runtime context created by this process."""
    from .runtime.executable import live_executables
    for exe in list(live_executables):
        try:
            exe.shutdown()
        except Exception:  # pragma: no cover
            pass


atexit.register(shutdown)
