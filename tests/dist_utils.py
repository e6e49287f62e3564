"""Helpers to run a function on several Gloo ranks (CPU) in child processes."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out[rank] = fn(rank, world, *args)
    except Exception:
        out[rank] = ("__error__", traceback.format_exc())
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world, *args):
    """Run ``fn(rank, world, *args)`` on ``world`` Gloo ranks; returns {rank: result}."""
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    out = mgr.dict()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    res = dict(out)
    for r in range(world):
        assert r in res, f"rank {r} produced no result"
        if isinstance(res[r], tuple) and len(res[r]) == 2 and res[r][0] == "__error__":
            raise AssertionError(f"rank {r} failed:\n{res[r][1]}")
    return res
