"""Failure handling on the host.

The reference aborts the MPI world through mpi4py on divergence
(``dl_code/pcode/utils/error_handler.py:37-47``).  Here failures are host-side
exceptions: a diverged loss, a peer that did not raise its flag inside the wait budget
(the gossip kernels return a status word instead of spinning forever), or a lost rank.
``abort`` tears the process group down so the surviving ranks' next collective fails
fast instead of hanging."""
from __future__ import annotations

import os
import sys
import traceback


class TrainingDiverged(RuntimeError):
    pass


class GossipTimeout(RuntimeError):
    """A peer did not publish its payload inside the wait budget."""

    def __init__(self, status: int, peer: int, step: int):
        super().__init__(f"gossip wait timed out (status={status}, peer={peer}, step={step})")
        self.status, self.peer, self.step = status, peer, step


class PeerLost(RuntimeError):
    def __init__(self, ranks):
        super().__init__(f"lost peers: {sorted(ranks)}")
        self.ranks = sorted(ranks)


def global_except_hook(exctype, value, tb):
    """Optional ``sys.excepthook``: print, tear down the process group, exit non-zero."""
    try:
        sys.stderr.write("\n*****************************************************\n")
        sys.stderr.write("Uncaught exception was detected on this rank.\n")
        traceback.print_exception(exctype, value, tb)
        sys.stderr.write("*****************************************************\n\n")
        sys.stderr.flush()
    finally:
        abort(exit_code=1)


def install_except_hook():
    sys.excepthook = global_except_hook


def abort(exit_code: int = 1):
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(exit_code)
