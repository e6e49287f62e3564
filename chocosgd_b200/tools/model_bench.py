"""Training-step benchmark for any vision architecture of the model zoo with CHOCO-SGD on a ring:
images/s over all GPUs, device-timed, synthetic data.

    # ResNet-50, 224 x 224, batch 128 per GPU, bf16 autocast, sign compression
    python -m chocosgd_b200.tools.model_bench --arch resnet50 --data imagenet --batch 128 --amp bf16 --comm_op sign
    python -m torch.distributed.run --nproc-per-node 8 -m chocosgd_b200.tools.model_bench --arch resnet50 ...
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--arch", default="resnet50")
    p.add_argument("--data", default="imagenet", help="imagenet (224 x 224, 1000 classes) or cifar10 / cifar100")
    p.add_argument("--batch", type=int, default=128)
    p.add_argument("--comm_op", default="sign")
    p.add_argument("--consensus_stepsize", type=float, default=0.45)
    p.add_argument("--amp", default="none", choices=("none", "bf16"))
    p.add_argument("--native_layers", default="auto")
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--no_graph", action="store_true")
    a = p.parse_args(argv)
    from ..config import get_args
    from ..models import define_model
    from ..ops import nn as native_nn
    from ..optim import define_optimizer
    from ..parallel.topology import Graph
    from ..train.engine import TrainStep

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    argv2 = ["--arch", a.arch, "--data", a.data, "--optimizer", "parallel_choco_v", "--comm_op", a.comm_op,
             "--graph_topology", "ring", "--n_mpi_process", str(world), "--lr", "0.1", "--momentum_factor", "0.9",
             "--use_nesterov", "True", "--weight_decay", "1e-4", "--consensus_stepsize", str(a.consensus_stepsize),
             "--batch_size", str(a.batch), "--gossip_impl", "fused"]
    if "compress" in a.comm_op:
        argv2 += ["--compress_ratio", "0.99"]
    if a.comm_op == "quantize_qsgd":
        argv2 += ["--quantize_level", "4", "--is_biased", "True"]
    conf = get_args(argv2)
    graph = Graph("ring", world, rank)
    torch.manual_seed(6)
    torch.backends.cudnn.benchmark = True
    native_nn.configure_native(a.native_layers)
    model = define_model(conf, graph, device=dev, verbose=False)
    opt = define_optimizer(conf, model, graph)
    hw, classes = (224, 1000) if a.data == "imagenet" else (32, 100 if a.data == "cifar100" else 10)
    g = torch.Generator().manual_seed(rank)
    xs = [torch.randn(a.batch, 3, hw, hw, generator=g).pin_memory() for _ in range(2)]
    ys = [torch.randint(0, classes, (a.batch,), generator=g).pin_memory() for _ in range(2)]
    step = TrainStep(model, torch.nn.CrossEntropyLoss(), opt, xs[0], ys[0], use_cuda_graph=not a.no_graph,
                     amp_dtype=torch.bfloat16 if a.amp == "bf16" else None)
    model.train()
    for i in range(max(a.warmup, 3)):
        step(xs[i % 2], ys[i % 2])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        loss = step(xs[i % 2], ys[i % 2])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    opt.finalize()
    opt.engine.check()
    if rank == 0:
        print(json.dumps({"bench": "model", "arch": a.arch, "data": a.data, "n_gpus": world, "batch_per_gpu": a.batch,
                          "images_per_s": a.batch * world * a.steps / (ms * 1e-3), "ms_per_step": ms / a.steps,
                          "loss": float(loss), "amp": a.amp, "comm_op": a.comm_op, "graph": step.use_graph,
                          "native_layers": a.native_layers, "includes": "pinned H2D copy of every batch",
                          "params": sum(p.numel() for p in model.parameters()),
                          "kernels_per_gossip_step": opt.engine.launches_per_step}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
