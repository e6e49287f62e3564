"""All-reduce of a flat fp32 buffer: the in-switch kernel (``parallel/nvls.py``: ``multimem.ld_reduce`` +
``multimem.st``) against the process group's ``all_reduce`` (NCCL), device time per call, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m chocosgd_b200.tools.allreduce_bench --sizes 262144,16777216,268435456

Bus bandwidth = 2 (n - 1) / n x bytes / time, the figure collective benchmarks quote."""
from __future__ import annotations

import argparse
import json
import os


def main(argv=None):
    import torch
    import torch.distributed as dist

    p = argparse.ArgumentParser()
    p.add_argument("--sizes", default="262144,4194304,67108864,268435456", help="elements (fp32)")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    a = p.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from ..parallel import nvls

    sizes = [int(s) for s in a.sizes.split(",")]
    ar = nvls.enable(max(sizes), device=dev)

    def timed(fn):
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t) * 1e3

    for n in sizes:
        x = torch.randn(n, device=dev)
        us_lib = timed(lambda: dist.all_reduce(x))
        row = {"bench": "allreduce", "n_gpus": world, "elements": n, "bytes": 4 * n, "library_us": round(us_lib, 2),
               "library_busbw_GBps": round(2 * (world - 1) / world * 4 * n / (us_lib * 1e-6) / 1e9, 1)}
        if ar is not None:
            us = timed(lambda: ar.reduce_(n, average=False))
            ar.check()
            row.update(multimem_us=round(us, 2),
                       multimem_busbw_GBps=round(2 * (world - 1) / world * 4 * n / (us * 1e-6) / 1e9, 1),
                       speedup=round(us_lib / us, 2))
        else:
            row["multimem"] = "unavailable: " + nvls.why_not()
        if rank == 0:
            print(json.dumps(row), flush=True)
        del x
    torch.cuda.synchronize()
    dist.barrier()
    nvls.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
