"""Process-group bootstrap: one process per GPU (NCCL) or per CPU rank (Gloo).

The reference initialises ``torch.distributed`` with MPI, or with NCCL/Gloo through a
``file://`` rendezvous and a 120 s timeout (``dl_code/main.py:26-44``).  Here the
rendezvous is taken from the launcher's environment (``RANK`` / ``WORLD_SIZE`` /
``MASTER_ADDR`` / ``MASTER_PORT``, as set by ``torch.distributed.run`` or by
``chocosgd_b200.run``), with the file rendezvous kept for ``--local_rank`` launches.
``backend mpi`` is mapped to NCCL (GPU) or Gloo (CPU): MPI is not part of this stack.
"""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist


def resolve_backend(backend: str, on_cuda: bool) -> str:
    if backend in ("nccl", "gloo"):
        if backend == "nccl" and not (on_cuda and torch.cuda.is_available()):
            return "gloo"
        return backend
    return "nccl" if (on_cuda and torch.cuda.is_available()) else "gloo"


def init_distributed_world(conf, timeout_s: float = 120.0) -> tuple:
    """-> (rank, world_size).  Idempotent."""
    if dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    env_world = int(os.environ.get("WORLD_SIZE", "0") or 0)
    n = env_world or int(conf.n_mpi_process)
    if env_world:
        rank = int(os.environ["RANK"])
    else:
        rank = int(conf.local_rank) if conf.local_rank is not None else 0
    conf.n_mpi_process = n
    backend = resolve_backend(conf.backend, conf.on_cuda)
    if n == 1 and not env_world:
        return 0, 1
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1)))
        torch.cuda.set_device(local)
    timeout = datetime.timedelta(seconds=timeout_s)
    if env_world:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend, rank=rank, world_size=n, timeout=timeout)
    else:
        dist_init_file = os.path.join(conf.checkpoint, "tmp", str(conf.timestamp), "dist_init")
        os.makedirs(os.path.dirname(dist_init_file), exist_ok=True)
        dist.init_process_group(
            backend, init_method="file://" + os.path.abspath(dist_init_file), rank=rank, world_size=n, timeout=timeout
        )
    return rank, n


def shutdown(collective: bool = True):
    """Tear the process group down.  ``collective=False``: the default group still counts a rank that
    is gone (an elastic run after a membership change), so nothing that waits for all of its ranks may
    run; the groups are dropped without a closing hand-shake."""
    if dist.is_available() and dist.is_initialized():
        from . import nvls

        if nvls.active() is not None:
            # no rank may drop its multicast binding while another rank's kernel can still use it
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            if collective:
                dist.barrier()
            nvls.close()
        if collective:
            dist.destroy_process_group()
        else:
            try:
                if torch.cuda.is_available():
                    torch.cuda.synchronize()
                dist.destroy_process_group()
            except Exception as e:  # a teardown that cannot complete must not fail a finished run
                print(f"[bootstrap] teardown without all ranks: {e!r}")


def heartbeat_check(store, rank: int, world_size: int, step: int, max_lag: int = 1_000_000, prefix: str = "hb"):
    """Host-side liveness: every rank publishes its step in the store; returns the ranks
    whose key says they left (``-1``).  Used between steps, never while a kernel or a
    collective is in flight."""
    store.set(f"{prefix}/{rank}", str(step))
    lost = []
    for r in range(world_size):
        if r == rank:
            continue
        try:
            v = int(store.get(f"{prefix}/{r}").decode()) if store.check([f"{prefix}/{r}"]) else step
        except Exception:
            v = step
        if v < 0:
            lost.append(r)
    return lost


def announce_leave(store, rank: int, prefix: str = "hb"):
    store.set(f"{prefix}/{rank}", "-1")
