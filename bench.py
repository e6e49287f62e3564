"""Headline benchmark: ResNet-20 (CIFAR shape, batch 128 per GPU, fp32) trained with
CHOCO-SGD on a ring, images/s over all GPUs.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...             # the unmodified reference
    python bench.py --model lstm ...                          # 2 x 650 LSTM language model, CHOCO + QSGD, tokens/s
    python bench.py --model resnet50 ...                      # ResNet-50 224 x 224, bf16 autocast, CHOCO + sign

For N > 1 launch one rank per GPU with ``python -m torch.distributed.run``.  Rank 0 prints
one JSON line.  Synthetic data (N(0,1) images, uniform labels), random-init weights.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# consensus step sizes inside the reference's tuning range [0.01, 0.5]; top-/random-1 % needs a small
# one (chocosgd_b200.tools.tune_consensus_stepsize: 0.012 - 0.04 on rings of 2 - 8 nodes)
GAMMA = {"compress_top_k": 0.02, "compress_random_k": 0.01, "sign": 0.45, "quantize_qsgd": 0.3}
QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

# The workloads of the benchmark configurations: the headline (ResNet-20, default), the LSTM language
# model and ResNet-50.  Each arm builds the same model family, optimizer and batch shapes.
WORKLOADS = {
    "resnet20": dict(
        metric="ResNet-20 CHOCO-ring images/s", unit="images/s", batch=128, items_per_sample=1, comm_op="compress_top_k",
        n_host_batches=16, dtype="fp32 (TF32 tensor-core convolutions, torch default)",
        data="synthetic N(0,1) 32x32x3 images, uniform labels, random-init weights",
        l2="per-step working set (activations + gradients, ~0.3 GB) exceeds the 126 MB L2"),
    "lstm": dict(
        metric="LSTM-2x650 CHOCO-ring tokens/s", unit="tokens/s", batch=32, items_per_sample=35, comm_op="quantize_qsgd",
        n_host_batches=8, dtype="fp32 (strict fp32 linear layers, torch default; cuDNN LSTM GEMMs TF32 in both arms)",
        data="synthetic uniform token ids over a 33278-word vocabulary, random-init weights",
        l2="per-step working set (28 M parameters x 5 state vectors + 149 MB of logits) exceeds the 126 MB L2"),
    "resnet50": dict(
        metric="ResNet-50 CHOCO-ring images/s", unit="images/s", batch=128, items_per_sample=1, comm_op="sign",
        n_host_batches=4, dtype="bf16 autocast (fp32 master weights and optimizer state)",
        data="synthetic N(0,1) 224x224x3 images, uniform labels over 1000 classes, random-init weights",
        l2="activations of one step (several GB) exceed the 126 MB L2"),
}


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=20)
    p.add_argument("--impl", default="ours", choices=("ours", "reference"))
    p.add_argument("--model", default="resnet20", choices=tuple(WORKLOADS))
    p.add_argument("--comm_op", default=None,
                   choices=("compress_top_k", "sign", "quantize_qsgd", "compress_random_k"))
    p.add_argument("--no_graph", action="store_true")
    p.add_argument("--trajectory", type=int, default=0,
                   help="no timing: run this many steps from the weights in --init_file (written by the 'ours' arm, "
                   "read by the reference arm) on the same batches and print loss and consensus error per step")
    p.add_argument("--init_file", default=os.path.join(tempfile.gettempdir(), "choco_trajectory_init.pt"))
    p.add_argument("--gossip_bucket_mb", type=float, default=None,
                   help="gossip launched per bucket of tensors during the backward pass (sign codec); default: "
                   "off")
    p.add_argument("--native_layers", default="auto", choices=("auto", "all", "on", "off", "bn", "conv"))
    a = p.parse_args()
    a.wl = WORKLOADS[a.model]
    if a.comm_op is None:
        a.comm_op = a.wl["comm_op"]
    return a


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs.

    ``nvidia-smi`` needs a second or more to come up on a multi-GPU machine, so the sampler is
    started before the warm-up steps; ``mark()`` (called at the start of the timed region) waits
    for its first line and remembers how many lines precede the region."""

    def __init__(self, enabled, gpu_index):
        self.proc, self.path, self.skip = None, None, 0
        if not enabled:
            return
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def _lines(self):
        try:
            with open(self.path) as fh:
                return sum(1 for _ in fh)
        except Exception:
            return 0

    def mark(self, wait_s=15.0):
        if self.proc is None:
            return
        t0 = time.time()
        while self._lines() == 0 and time.time() - t0 < wait_s:
            time.sleep(0.05)
        self.skip = self._lines()

    def samples_in_region(self):
        return max(0, self._lines() - self.skip) if self.proc is not None else 0

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for n_line, line in enumerate(open(self.path)):
                if n_line < self.skip:
                    continue
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                for name, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            out = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


def init_dist(n):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1 or n > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        import datetime

        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=90))
    return rank, world, local


def host_batches(rank, model):
    """Pinned host batches of the workload's shape (the end-to-end region copies one per step)."""
    wl = WORKLOADS[model]
    g = torch.Generator().manual_seed(1000 + rank)
    n, b = wl["n_host_batches"], wl["batch"]
    if model == "lstm":
        xs = [torch.randint(0, 33278, (35, b), generator=g).pin_memory() for _ in range(n)]
        ys = [torch.randint(0, 33278, (35, b), generator=g).pin_memory() for _ in range(n)]
        return xs, ys
    hw, classes = (224, 1000) if model == "resnet50" else (32, 10)
    xs = [torch.randn(b, 3, hw, hw, generator=g).pin_memory() for _ in range(n)]
    ys = [torch.randint(0, classes, (b,), generator=g).pin_memory() for _ in range(n)]
    return xs, ys


def barrier_sync(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms, world):
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return ms


def timed(fn, steps, world, quiesce=None):
    """K calls of fn(i) bracketed by barrier + synchronize, CUDA events, max over ranks.

    ``quiesce`` runs before each barrier: an arm that communicates from a helper thread must
    have no point-to-point call in flight while this thread issues a collective on the same
    NCCL communicator (the two would be enqueued in different orders on different ranks)."""
    if quiesce is not None:
        quiesce()
    barrier_sync(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if quiesce is not None:
        quiesce()
    barrier_sync(world)
    return max_over_ranks(ms, world)


def keep_load_until_sampled(sampler, fn, world, quiesce=None, want=3, limit_s=6.0):
    """A short timed region can end before nvidia-smi (one line per 100 ms) has printed three
    lines: keep running the same step, untimed, until it has.  Rank 0 owns the sampler and
    decides; all ranks run the same number of extra steps (the steps exchange payloads)."""
    t0 = time.time()
    while True:
        more = 1 if (sampler.proc is not None and sampler.samples_in_region() < want
                     and time.time() - t0 < limit_s) else 0
        if world > 1:
            flag = torch.tensor([more], dtype=torch.int32, device="cuda")
            if quiesce is not None:
                quiesce()
            dist.broadcast(flag, 0)
            more = int(flag.item())
        if not more:
            return
        for i in range(20):
            fn(i)
        torch.cuda.synchronize()


def trajectory(args, rank, world, step_fn, flat_fn):
    """Loss of rank 0 and consensus error sqrt(mean_i ||x_i - x_bar||^2) after every step; one JSON line."""
    rows = []
    for i in range(args.trajectory):
        loss = step_fn(i)
        torch.cuda.synchronize()
        x = flat_fn().detach().float().clone()
        mean = x.clone()
        if world > 1:
            dist.all_reduce(mean)
            mean /= world
        err = (x - mean).pow(2).sum()
        if world > 1:
            dist.all_reduce(err)
        rows.append((float(loss), float((err / world).sqrt())))
    if rank == 0:
        emit({"trajectory": args.impl, "model": args.model, "comm_op": args.comm_op, "n_gpus": world,
              "loss": [round(r[0], 5) for r in rows], "consensus_error": [round(r[1], 6) for r in rows]})
    return None


def run_ours(args, rank, world, local):
    from chocosgd_b200.config import get_args
    from chocosgd_b200.models import define_model
    from chocosgd_b200.optim import define_optimizer
    from chocosgd_b200.parallel.topology import Graph
    from chocosgd_b200.train.engine import TrainStep
    from chocosgd_b200.train.metrics import Metrics
    from chocosgd_b200.ops import nn as native_nn

    device = torch.device("cuda", local)
    wl, batch = args.wl, args.wl["batch"]
    argv = ["--optimizer", "parallel_choco_v", "--comm_op", args.comm_op, "--graph_topology", "ring",
            "--n_mpi_process", str(world), "--consensus_stepsize", str(GAMMA[args.comm_op]),
            "--batch_size", str(batch), "--gossip_impl", "fused"]
    if args.model == "lstm":
        argv += ["--arch", "rnn_lm", "--lr", "2.5", "--momentum_factor", "0.0", "--weight_decay", "0",
                 "--rnn_n_hidden", "650", "--rnn_n_layers", "2", "--drop_rate", "0.4", "--rnn_clip", "0.4"]
    else:
        argv += ["--arch", args.model, "--data", "imagenet" if args.model == "resnet50" else "cifar10", "--lr", "0.1",
                 "--momentum_factor", "0.9", "--use_nesterov", "True", "--weight_decay", "1e-4"]
    if "compress" in args.comm_op:
        argv += ["--compress_ratio", "0.99"]
    if args.comm_op == "quantize_qsgd":
        argv += ["--quantize_level", "4", "--is_biased", "True"]
    conf = get_args(argv)
    graph = Graph("ring", world, rank)
    torch.manual_seed(6)
    torch.backends.cudnn.benchmark = True
    native_nn.configure_native("auto" if args.native_layers == "on" else args.native_layers)
    from chocosgd_b200.ops import _lib as native_lib

    pdl = native_lib.configure_pdl(conf.pdl, bf16=args.model == "resnet50")   # before the library's first launch
    loader = {"n_tokens": 33278} if args.model == "lstm" else None
    model = define_model(conf, graph, data_loader=loader, device=device, verbose=False)
    if args.trajectory:
        if rank == 0:
            os.makedirs(os.path.dirname(args.init_file), exist_ok=True)
            torch.save({k: v.detach().cpu() for k, v in model.state_dict().items()}, args.init_file)
        if world > 1:
            dist.barrier()
        model.load_state_dict(torch.load(args.init_file, map_location=device))   # every rank: rank 0's weights
    optimizer = define_optimizer(conf, model, graph)
    criterion = torch.nn.CrossEntropyLoss()
    xs, ys = host_batches(rank, args.model)
    nb = len(xs)
    kw = {}
    if args.model == "lstm":
        kw = dict(metrics=Metrics(model, "language_modeling"), clip_grad_norm=conf.rnn_clip,
                  hidden=tuple(h.to(device) for h in model.init_hidden(batch)))
    elif args.model == "resnet50":
        kw = dict(metrics=Metrics(model), amp_dtype=torch.bfloat16)
    else:
        kw = dict(metrics=Metrics(model))
    # (bucketed launches measured 27.41 ms against 27.31 ms per ResNet-50 step on one GPU: off unless asked for)
    bucket_mb = args.gossip_bucket_mb if args.gossip_bucket_mb is not None else 0.0
    step = TrainStep(model, criterion, optimizer, xs[0], ys[0], use_cuda_graph=not args.no_graph,
                     gossip_bucket_mb=bucket_mb, **kw)
    model.train()
    if args.trajectory:
        return trajectory(args, rank, world, lambda i: step(xs[i % nb], ys[i % nb]), lambda: optimizer.arena.x)
    loss_host = torch.zeros(args.steps + args.warmup + 8, dtype=torch.float32).pin_memory()

    # warm-up: graph capture + W untimed steps through the public call
    sampler = ClockSampler(rank == 0, local)
    for i in range(max(args.warmup, 3)):
        step(xs[i % nb], ys[i % nb])
    torch.cuda.synchronize()
    optimizer.check()
    sampler.mark()

    # (1) device-timed steps: the batch is already in the static device buffers
    dev_ms = timed(lambda i: step(), args.steps, world)

    # (2) end to end through the public API: pinned host batch -> device, step, loss -> host
    def e2e(i):
        loss = step(xs[i % nb], ys[i % nb])
        loss_host[i:i + 1].copy_(loss.reshape(1), non_blocking=True)

    e2e_ms = timed(e2e, args.steps, world)
    keep_load_until_sampled(sampler, lambda i: step(), world)
    clocks = sampler.stop()
    optimizer.finalize()
    optimizer.check()
    losses = loss_host[:args.steps]
    assert torch.isfinite(losses).all(), "training diverged"
    # kernels of the native library per step: counted by the Python wrappers while the step was
    # captured (convolutions, batch-norm, weight gradients, loss, gossip); library kernels excluded
    per_step = step.kernel_launches_per_step or optimizer.engine.launches_per_step
    launches = per_step * args.steps
    return dev_ms, e2e_ms, clocks, launches, float(losses[-1]), step.h2d_bytes, {
        "graph": step.use_graph, "native_layers": args.native_layers,
        "gossip_kernels_per_step": optimizer.engine.launches_per_step, "native_kernels_per_step": per_step,
        "gossip_buckets": len(optimizer.bucket_plan(step._bucket_bytes)) if step._bucket_bytes else 0,
        "programmatic_dependent_launch": bool(pdl)}


def run_reference(args, rank, world, local):
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ref

    if not ref.available():
        return None
    device = torch.device("cuda", local)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    torch.backends.cudnn.benchmark = True
    batch = args.wl["batch"]
    state = ref.build(rank, world, args.comm_op, batch, device, GAMMA[args.comm_op], model_name=args.model,
                      init_state=args.init_file if args.trajectory else None)
    xs, ys = host_batches(rank, args.model)
    nb = len(xs)
    out = {}
    if args.model == "lstm":
        out["hidden"] = state[1].init_hidden(batch)

    def it(i):
        if args.model == "lstm":
            out["loss"], out["hidden"] = ref.train_iteration_lm(*state, xs[i % nb], ys[i % nb], it.n, out["hidden"])
        else:
            out["loss"], _ = ref.train_iteration(*state, xs[i % nb], ys[i % nb], it.n,
                                                 amp_dtype=torch.bfloat16 if args.model == "resnet50" else None)
        it.n += 1

    it.n = 0
    if args.trajectory:
        def flat():
            return torch.cat([p.data.reshape(-1) for p in state[1].parameters()])

        def one(i):
            it(i)
            ref.finish(state)   # the helper thread's exchange must not be in flight under the collectives below
            return out["loss"]

        res = trajectory(args, rank, world, one, flat)
        ref.finish(state)
        return res
    sampler = ClockSampler(rank == 0, local)
    for i in range(max(args.warmup, 3)):
        it(i)
    torch.cuda.synchronize()
    sampler.mark()
    ms = timed(it, args.steps, world, quiesce=lambda: ref.finish(state))
    keep_load_until_sampled(sampler, it, world, quiesce=lambda: ref.finish(state))
    clocks = sampler.stop()
    ref.finish(state)
    h2d = xs[0].numel() * xs[0].element_size() + ys[0].numel() * ys[0].element_size()
    return ms, ms, clocks, 0, out["loss"], h2d, {}


_JSON_OUT = None


def claim_stdout():
    """Keep the real stdout for the ONE JSON line: libraries that write to file descriptor 1
    themselves (NCCL prints its version there) are sent to stderr from here on."""
    global _JSON_OUT
    sys.stdout.flush()
    _JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(obj):
    print(json.dumps(obj), file=_JSON_OUT if _JSON_OUT is not None else sys.stdout, flush=True)


def main():
    args = parse()
    claim_stdout()
    if not torch.cuda.is_available():
        emit({"impl": args.impl, "unavailable": "no CUDA device"})
        return
    rank, world, local = init_dist(args.gpus)
    if args.trajectory:
        (run_reference if args.impl == "reference" else run_ours)(args, rank, world, local)
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
        return
    if args.impl == "reference":
        try:
            res = run_reference(args, rank, world, local)
        except Exception as e:  # the reference arm must never take the bench down
            res = ("error", repr(e)[:300])
        if res is None or res[0] == "error":
            if rank == 0:
                why = "reference not installed under baseline/_ref" if res is None else res[1]
                emit({"impl": "reference", "unavailable": why})
            return
    else:
        res = run_ours(args, rank, world, local)
    dev_ms, e2e_ms, clocks, launches, last_loss, h2d, extra = res
    if rank == 0:
        wl = args.wl
        items = wl["batch"] * wl["items_per_sample"] * world * args.steps
        config = {"model": {"resnet20": "resnet20", "resnet50": "resnet50", "lstm": "lstm-2x650-tied"}[args.model],
                  "global_batch": wl["batch"] * world, "seq_len": 35 if args.model == "lstm" else None,
                  "parallelism": f"gossip-dp{world} ring", "optimizer": "CHOCO-SGD", "comm_op": args.comm_op,
                  "consensus_stepsize": GAMMA[args.comm_op], "l2": wl["l2"]}
        if "compress" in args.comm_op:
            config["compress_ratio"] = 0.99
        if args.comm_op == "quantize_qsgd":
            config["quantize_level"] = 4
        if args.model == "lstm":
            config.update({"momentum": 0.0, "weight_decay": 0.0, "grad_clip": 0.4, "dropout": 0.4, "vocab": 33278})
        else:
            config.update({"nesterov": 0.9, "weight_decay": 1e-4})
        line = {
            "metric": wl["metric"], "value": items / (dev_ms * 1e-3), "unit": wl["unit"],
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl["dtype"], "data": wl["data"],
            "impl": args.impl,
            "config": config,
            "impl_detail": extra,
            "clocks": clocks,
            "e2e": {"value": items / (e2e_ms * 1e-3), "unit": wl["unit"], "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches,
            "last_loss": last_loss,
        }
        emit(line)
    if dist.is_initialized():
        try:
            torch.cuda.synchronize()
            dist.barrier()
            dist.destroy_process_group()
        except Exception as e:  # a failing teardown must not turn a measured run into an error
            print(f"[bench] teardown: {e!r}", file=sys.stderr)


if __name__ == "__main__":
    main()
