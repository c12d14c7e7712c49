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
from typing import List, Optional, Tuple

import torch

from . import state

_log = logging.getLogger("multimesh_jax_b200")


def init(cpus: int = 0, gpus: int = 0, fbmem: int = 8000, sysmem: int = 4000, zcmem: int = 32, debug: int = 0,
         network: str = "none", kthreads: int = 0, profile: bool = False, distributed: bool = False,
         dump: Optional[str] = None, dump_all_passes: bool = False, realm_argv: Optional[List[str]] = None,
         coordinator_address: Optional[str] = None, num_processes: Optional[int] = None,
         process_id: Optional[int] = None, local_device_ids: Optional[List[int]] = None,
         initialization_timeout: int = 300, cluster_detection_method: Optional[str] = None,
         coordinator_bind_address: Optional[str] = None) -> state.StartupConfig:
    """Process start-up (counterpart of ``jax_plugins/multimesh/init.py:12-136``). With
    ``distributed=True`` the process joins the job: rank, world size and local device come from the
    explicit arguments, else from the launcher named by ``cluster_detection_method`` (``"torchrun"``,
    ``"slurm"``, ``"ompi"``; None = the first of them whose variables are set). The coordinator is
    ``coordinator_address`` (``host:port``); ``coordinator_bind_address`` is the address rank 0's
    rendezvous store listens on when it differs from the address the others connect to."""
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
            found = detect_cluster(cluster_detection_method)
            if num_processes is None and found is not None:
                num_processes = found[1]
            if process_id is None and found is not None:
                process_id = found[0]
            if num_processes is not None:
                os.environ.setdefault("WORLD_SIZE", str(num_processes))
            if process_id is not None:
                os.environ.setdefault("RANK", str(process_id))
            use_cuda = torch.cuda.is_available() and gpus != 0
            if use_cuda:
                fallback = (local_device_ids or [found[2] if found is not None else 0])[0]
                local = int(os.environ.get("LOCAL_RANK", fallback))
                torch.cuda.set_device(local)
            store = None
            timeout = datetime.timedelta(seconds=initialization_timeout)
            if coordinator_bind_address and int(os.environ.get("RANK", "0")) == 0:
                # rank 0 listens on the bind address; the others reach it through MASTER_ADDR
                host, _, port = coordinator_bind_address.partition(":")
                store = dist.TCPStore(host or "0.0.0.0", int(port or os.environ.get("MASTER_PORT", "29500")),
                                      int(os.environ["WORLD_SIZE"]), True, timeout)
            if store is not None:
                dist.init_process_group("nccl" if use_cuda else "gloo", store=store, timeout=timeout,
                                        rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
            else:
                dist.init_process_group("nccl" if use_cuda else "gloo", timeout=timeout)
    cfg.initialized = True
    return cfg


_LAUNCHERS = {
    "torchrun": ("RANK", "WORLD_SIZE", "LOCAL_RANK"),
    "slurm": ("SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID"),
    "ompi": ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK"),
}


def detect_cluster(method: Optional[str] = None) -> Optional[Tuple[int, int, int]]:
    """(process id, number of processes, local id) from the launcher's environment, or None."""
    if method is not None and method not in _LAUNCHERS:
        raise ValueError(f"unknown cluster_detection_method {method!r}; expected one of {sorted(_LAUNCHERS)}")
    for name in ([method] if method else list(_LAUNCHERS)):
        rank, world, local = _LAUNCHERS[name]
        if rank in os.environ and world in os.environ:
            return int(os.environ[rank]), int(os.environ[world]), int(os.environ.get(local, "0"))
    if method is not None:
        raise RuntimeError(f"cluster_detection_method={method!r}: its environment variables are not set")
    return None


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
