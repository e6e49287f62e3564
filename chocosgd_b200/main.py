"""Per-rank entry point: ``python -m chocosgd_b200.main --arch resnet20 --optimizer parallel_choco ...``

Order of ``dl_code/main.py:47-149``: process group -> graph / seeds / checkpoint dir / logger
-> timer -> dataset -> model (rank-0 weights everywhere) -> optimizer -> scheduler ->
optional resume -> criterion / metrics / best tracker -> save arguments -> train."""
from __future__ import annotations

import sys

import numpy as np
import torch

from . import config as cfg
from .data import define_dataset
from .models import define_model
from .optim import define_optimizer
from .parallel import bootstrap
from .parallel.topology import define_graph_topology
from .train.loops import train_and_validate
from .train.metrics import Metrics
from .train.scheduler import Scheduler
from .utils import checkpoint as ckpt
from .utils.logging import Logger, display_args
from .utils.stat_tracker import BestPerf
from .utils.timer import Timer


def init_config(conf, rank, world):
    run = cfg.RunState()
    world_ids = conf.world if conf.world is not None else ",".join(str(i % max(torch.cuda.device_count(), 1))
                                                                 for i in range(world * conf.n_sub_process))
    on_cuda = bool(conf.on_cuda and torch.cuda.is_available())
    graph = define_graph_topology(
        conf.graph_topology, world=world_ids, n_mpi_process=world, n_sub_process=conf.n_sub_process,
        comm_device=conf.comm_device, on_cuda=on_cuda, rank=rank,
    )
    run.graph = graph
    run.is_centralized = conf.graph_topology == "complete"
    if conf.n_sub_process > 1:
        conf.batch_size = conf.batch_size * conf.n_sub_process
    torch.manual_seed(conf.manual_seed)
    np.random.seed(conf.manual_seed)
    if on_cuda:
        from .ops import _lib as native_lib

        native_lib.configure_pdl(conf.pdl, bf16=conf.dtype == "bf16")
        torch.cuda.manual_seed(conf.manual_seed)
        # the library convolutions that remain pick their algorithm by measurement, with or without
        # --train_fast (the reference ties cudnn.deterministic to that flag, dl_code/main.py:177-179; the
        # native kernels are reproducible either way)
        torch.backends.cudnn.benchmark = True
    ckpt.init_checkpoint(conf, graph, run)
    run.logger = Logger(run.checkpoint_dir)
    display_args(conf, graph)
    return run, graph


def main(conf):
    cfg.validate(conf)
    rank, world = bootstrap.init_distributed_world(conf)
    run, graph = init_config(conf, rank, world)
    device = None
    if graph.on_cuda:
        device = torch.device("cuda", torch.cuda.current_device() if world > 1 else graph.device[0] % torch.cuda.device_count())
        torch.cuda.set_device(device)
    run.timer = Timer(
        verbosity_level=1 if conf.track_time and not conf.train_fast else 0,
        log_fn=run.logger.log_metric, on_cuda=graph.on_cuda,
    )
    if graph.on_cuda:
        from .ops import nn as native_nn

        native_nn.configure_native(getattr(conf, "native_layers", "auto"))
    data_loader = define_dataset(conf, graph, run, device=device)
    model = define_model(conf, graph, data_loader=data_loader, device=device)
    optimizer = define_optimizer(conf, model, graph)
    scheduler = Scheduler(conf, graph, run)
    ckpt.maybe_resume_from_checkpoint(conf, graph, run, model, optimizer, scheduler)
    criterion = torch.nn.CrossEntropyLoss(reduction="mean")
    if "rnn_lm" in conf.arch:
        metrics = Metrics(model, task="language_modeling")
        best = BestPerf(best_perf=run.best_perf, larger_is_better=False)
    else:
        metrics = Metrics(model, task="classification")
        best = BestPerf(best_perf=run.best_perf, larger_is_better=True)
    scheduler.set_best_tracker(best)
    if (world > 1 and graph.on_cuda and getattr(conf, "nvls", "auto") != "off" and not conf.elastic
            and getattr(optimizer, "arena", None) is not None):
        # flat all-reduces (averaged-model evaluation, centralized aggregation) run inside the NVSwitch
        # where the system has NVLink multicast; never in elastic runs, where a rank may leave
        from .parallel import nvls

        if nvls.enable(optimizer.arena.x.numel(), device=optimizer.arena.x.device) is None and rank == 0:
            print(f"[nvls] in-switch all-reduce not used: {nvls.why_not()}")
    if conf.elastic and world > 1:
        import torch.distributed as dist

        from .parallel.elastic import Membership

        run.membership = Membership(dist.distributed_c10d._get_default_store(), rank, list(range(world)),
                                    stale_after_s=conf.heartbeat_stale_s)
    ckpt.save_arguments(conf, graph, run)
    try:
        train_and_validate(conf, graph, run, model, criterion, scheduler, optimizer, metrics, data_loader, device)
    finally:
        run.logger.save_json()
    # after a membership change the default group still counts the rank that left: no collective on it
    bootstrap.shutdown(collective=run.extras.get("lost_ranks") is None)
    return run, scheduler


if __name__ == "__main__":
    main(cfg.get_args(sys.argv[1:]))
