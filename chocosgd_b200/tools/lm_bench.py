"""Language-model benchmark: 2-layer LSTM (650 hidden, vocab 33 278, tied weights, dropout 0.4, bptt 35,
batch 32 per GPU, fp32) trained with CHOCO-SGD + QSGD on a ring, tokens/s over all GPUs.

    python -m chocosgd_b200.tools.lm_bench --steps 50
    python -m torch.distributed.run --nproc-per-node 8 -m chocosgd_b200.tools.lm_bench
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--no_graph", action="store_true")
    p.add_argument("--native", default="off", help="comma list of native layer kinds (ce, lstm, linear) or off")
    p.add_argument("--tf32_matmul", action="store_true",
                   help="let the library run the fp32 decoder / embedding GEMMs on TF32 tensor cores (PyTorch keeps "
                        "them on fp32 FMA units by default, which is 3.1 of the 6.2 ms step; the LSTM's own GEMMs "
                        "are TF32 either way)")
    a = p.parse_args(argv)
    torch.backends.cuda.matmul.allow_tf32 = bool(a.tf32_matmul)
    from ..config import get_args
    from ..models import define_model
    from ..optim import define_optimizer
    from ..parallel.topology import Graph
    from ..train.engine import TrainStep
    from ..train.metrics import Metrics

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    B, T, V = 32, 35, 33278
    conf = get_args(["--arch", "rnn_lm", "--optimizer", "parallel_choco_v", "--comm_op", "quantize_qsgd",
                     "--quantize_level", "4", "--is_biased", "True", "--graph_topology", "ring",
                     "--n_mpi_process", str(world), "--lr", "2.5", "--momentum_factor", "0.0", "--weight_decay", "0",
                     "--consensus_stepsize", "0.3", "--rnn_n_hidden", "650", "--rnn_n_layers", "2", "--drop_rate", "0.4",
                     "--rnn_clip", "0.4", "--batch_size", str(B), "--gossip_impl", "fused"])
    graph = Graph("ring", world, rank)
    torch.manual_seed(6)
    if a.native != "off":
        from ..ops import nn as native_nn

        native_nn.set_native(True, which=tuple(a.native.split(",")))
    model = define_model(conf, graph, data_loader={"n_tokens": V}, device=dev, verbose=False)
    opt = define_optimizer(conf, model, graph)
    g = torch.Generator().manual_seed(rank)
    xs = [torch.randint(0, V, (T, B), generator=g).pin_memory() for _ in range(8)]
    ys = [torch.randint(0, V, (T, B), generator=g).pin_memory() for _ in range(8)]
    hidden = tuple(h.to(dev) for h in model.init_hidden(B))
    step = TrainStep(model, torch.nn.CrossEntropyLoss(), opt, xs[0], ys[0], metrics=Metrics(model, "language_modeling"),
                     use_cuda_graph=not a.no_graph, clip_grad_norm=conf.rnn_clip, hidden=hidden)
    model.train()
    for i in range(max(a.warmup, 3)):
        step(xs[i % 8], ys[i % 8])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        loss = step(xs[i % 8], ys[i % 8])
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
        print(json.dumps({"bench": "lstm_lm", "n_gpus": world, "tokens_per_s": B * T * world * a.steps / (ms * 1e-3),
                          "ms_per_step": ms / a.steps, "loss": float(loss), "graph": step.use_graph, "native": a.native, "tf32_matmul": bool(a.tf32_matmul),
                          "kernels_per_step": opt.engine.launches_per_step, "comm_op": "quantize_qsgd 4 bit",
                          "params": sum(p.numel() for p in model.parameters())}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
