"""Training / validation loops for vision and language models.

Skeleton of ``dl_code/pcode/distributed_running_cv.py:23-258`` and
``dl_code/pcode/distributed_running_nlp.py:23-242``: barrier per epoch, per batch
``scheduler.step`` -> load batch -> forward / backward -> ``optimizer.step`` -> train record;
at integer epochs divergence guard, validation (local model, and the world-averaged model
with the L2 distance when ``--evaluate_consensus`` on a non-complete graph), checkpoint,
optional consensus evaluation on the full training set, stop check; optional reshuffle.

The hot path differs on purpose: one ``TrainStep`` call per batch (CUDA-graph replay with
the fused optimizers), loss / accuracy stay on the device and are read back in bulk every
``summary_freq`` steps instead of three ``.item()`` syncs per step."""
from __future__ import annotations

import copy
import gc
import math
import time

import torch
import torch.distributed as dist

from ..data import define_dataset, load_data_batch
from ..utils import checkpoint as ckpt
from ..utils.auxiliary import get_model_difference
from ..utils.error_handler import TrainingDiverged
from ..utils.logging import display_best_test_stat, display_test_stat, display_training_stat
from ..utils.stat_tracker import RuntimeTracker
from .engine import TrainStep


def _barrier(group=None):
    if dist.is_available() and dist.is_initialized():
        dist.barrier(group=group)


class _Elastic:
    """Membership checks between training steps and the recovery after a rank was lost.

    Every ``heartbeat_every`` steps (and whenever a bounded device-side wait ran out) the ranks
    compare heartbeats; survivors agree on who is gone, form a new process group and graph, and
    rebuild the optimizer's transports.  Nothing of this runs while a kernel or a collective of
    this rank is in flight: the stream is synchronised first."""

    def __init__(self, conf, run):
        self.conf, self.run, self.m = conf, run, run.membership
        self.leave_rank, self.leave_step = None, None
        if conf.leave_at_step:
            r, s = conf.leave_at_step.split(":")
            self.leave_rank, self.leave_step = int(r), int(s)

    def wants_to_leave(self, global_rank, step) -> bool:
        return self.leave_rank == global_rank and step >= self.leave_step

    def leave(self, optimizer):
        optimizer.finalize()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.m.leave()

    def lost_now(self, optimizer, step, force=False):
        """-> global ranks lost, or [] (cheap: one store write; reads only at check points)."""
        from ..utils.error_handler import GossipTimeout

        self.m.beat(step)
        timed_out = None
        if force or step % max(1, self.conf.heartbeat_every) == 0:
            try:
                optimizer.check()
            except GossipTimeout as e:
                timed_out = e
            lost = self.m.lost()
            if timed_out is not None and not lost:
                # a peer stopped publishing payloads: give its heartbeat the chance to go stale
                deadline = time.time() + (self.m.stale_after_s or 5.0) + 1.0
                while not lost and time.time() < deadline:
                    time.sleep(0.1)
                    lost = self.m.lost()
                if not lost:
                    raise timed_out
            return lost
        return []

    def after_failure(self, error):
        """A step failed (a send to a peer that is gone, a bounded wait that ran out): the ranks lost
        according to the membership record, waiting up to the staleness limit for it to show one;
        re-raises ``error`` when nobody is missing (the failure was something else)."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        deadline = time.time() + (self.m.stale_after_s or 5.0) + 1.0
        lost = self.m.lost()
        while not lost and time.time() < deadline:
            time.sleep(0.1)
            lost = self.m.lost()
        if not lost:
            raise error
        return lost

    def recover(self, seen_lost, graph, model, optimizer, scheduler):
        from ..parallel.elastic import rebuild_optimizer

        if torch.cuda.is_available():
            torch.cuda.synchronize()
        lost, resume_step = self.m.agree(seen_lost, scheduler.local_index)
        scheduler.local_index = resume_step      # survivors noticed the loss at different steps
        backend = dist.get_backend() if dist.is_initialized() else None
        new_graph, group = self.m.regroup(graph, lost, backend=backend)
        self.run.group, self.run.graph = group, new_graph
        self.run.extras["lost_ranks"] = sorted(set(self.run.extras.get("lost_ranks", [])) | set(lost))
        new_opt = rebuild_optimizer(self.conf, model, optimizer, new_graph, group)
        self.run.logger.log(f"lost ranks {lost}: continuing on {new_graph.n_nodes} nodes as rank {new_graph.rank}")
        return new_graph, new_opt


class _PendingRecords:
    """Per-step training records whose numbers are still on the device."""

    def __init__(self):
        self.meta, self.vals = [], []

    def add(self, meta, loss, perf):
        self.meta.append(meta)
        self.vals.append(torch.cat([loss.reshape(1), perf.reshape(-1)]).clone())

    def flush(self, logger, graph, tracker, names, display_every):
        if not self.meta:
            return
        vals = torch.stack(self.vals).cpu()
        for i, (meta, row) in enumerate(zip(self.meta, vals)):
            tracker.update_metrics([float(v) for v in row], n_samples=meta["n"])
            sch = meta["sched"]
            display_training_stat(logger, graph, sch, tracker, meta["bits"],
                                  display=(i == len(self.meta) - 1) or display_every)
        self.meta, self.vals = [], []


class _SchedView:
    def __init__(self, s):
        self.epoch_, self.local_index = s.epoch_, s.local_index


def inference(model, criterion, metrics, _input, _target, tracker=None, hidden=None):
    if hidden is not None:
        output, hidden = model(_input, hidden)
        loss = criterion(output.reshape(-1, output.size(-1)), _target.reshape(-1))
        perf = metrics.evaluate(loss, output.reshape(-1, output.size(-1)), _target.reshape(-1))
    else:
        output = model(_input)
        loss = criterion(output, _target)
        perf = metrics.evaluate(loss, output, _target)
    if tracker is not None:
        tracker.update_metrics([loss.detach()] + [p for p in perf], n_samples=_input.size(0))
    return loss, hidden


def _world_average(conf, run, optimizer, x):
    """The world-averaged flat parameters: in the NVSwitch (``parallel/nvls.py``) when the system has
    multicast and no rank may leave (not ``--elastic``, whole-world group), else the group's all-reduce."""
    from ..parallel import nvls

    group = getattr(run, "group", None)
    if getattr(conf, "nvls", "auto") != "off" and not getattr(conf, "elastic", False) and group is None:
        ar = nvls.enable(x.numel(), device=x.device)
        if ar is not None:
            out = ar.all_reduce(x, average=True).clone()
            torch.cuda.current_stream(x.device).synchronize()
            ar.check()
            return out
    return optimizer.world_aggregator._agg(x.clone(), op="avg")


def validate(conf, graph, run, model, optimizer, criterion, scheduler, metrics, data_loader, label="local_model",
             force_evaluate_on_averaged_model=True, device=None, rank_slice=None):
    is_nlp = "rnn_lm" in conf.arch

    def _evaluate(_model, label):
        tracker = RuntimeTracker(metrics.metric_names, on_cuda=graph.on_cuda, world_aggregator=optimizer.world_aggregator)
        _model.eval()
        hidden = _model.init_hidden(conf.batch_size) if is_nlp else None
        with torch.no_grad():
            for _input, _target in data_loader["val_loader"]:
                if is_nlp:
                    _input, _target = _input[:, rank_slice], _target[:, rank_slice]
                    if _input.size(1) != conf.batch_size:
                        continue
                _input, _target = load_data_batch(device, _input, _target)
                _, hidden = inference(_model, criterion, metrics, _input, _target, tracker, hidden)
                if is_nlp:
                    hidden = _model.repackage_hidden(hidden)
        display_test_stat(run.logger, graph, scheduler, tracker, label)
        return tracker.evaluate_global_metrics()

    if (conf.graph_topology != "complete" and not conf.train_fast and conf.evaluate_consensus
            and force_evaluate_on_averaged_model):
        arena = getattr(optimizer, "arena", None)
        if arena is not None and arena.x.is_cuda:
            # flat arena: ONE all-reduce gives the world-averaged parameters, the distance kernel the
            # consensus error ||x_i - x_bar||_2, and the averaged model is evaluated in place (the
            # local parameters are put back afterwards) - no model copy, no per-tensor collectives
            from ..parallel.exchange import sq_distance

            optimizer.finalize()
            x_local = arena.x.clone()
            x_bar = _world_average(conf, run, optimizer, arena.x)
            distance = float(sq_distance(x_local, x_bar).sqrt())
            arena.x.copy_(x_bar)
            try:
                _evaluate(model, label="averaged_model")
            finally:
                arena.x.copy_(x_local)
        else:
            copied = copy.deepcopy(model)
            optimizer.world_aggregator.agg_model(copied, op="avg")
            _evaluate(copied, label="averaged_model")
            distance = get_model_difference(model, copied)
        run.logger.log_metric(
            name="stat",
            values={"rank": graph.rank, "epoch": scheduler.epoch_, "distance": distance},
            tags={"split": "test", "type": "averaged_model"},
        )
    return _evaluate(model, label=label)


def do_validate(conf, graph, run, model, optimizer, criterion, scheduler, metrics, data_loader, device, rank_slice=None):
    print("Enter validation phase.")
    optimizer.finalize()
    performance = validate(conf, graph, run, model, optimizer, criterion, scheduler, metrics, data_loader,
                           device=device, rank_slice=rank_slice)
    perf0 = performance[0]
    scheduler.best_tracker.update(perf0, scheduler.epoch_)
    display_best_test_stat(run.logger, graph, scheduler)
    if not conf.train_fast:
        ckpt.save_to_checkpoint(
            run,
            {
                "arch": conf.arch,
                "current_epoch": scheduler.epoch,
                "local_index": scheduler.local_index,
                "best_perf": scheduler.best_tracker.best_perf,
                "optimizer": optimizer.state_dict(),
                "state_dict": model.state_dict(),
            },
            scheduler.best_tracker.is_best,
            dirname=run.checkpoint_dir,
            filename="checkpoint.pth.tar",
            save_all=conf.save_all_models,
        )
    print("Finished validation.")
    return performance


def train_and_validate(conf, graph, run, model, criterion, scheduler, optimizer, metrics, data_loader, device=None):
    """Run training until the stop criterion; returns the scheduler (with best_tracker)."""
    is_nlp = "rnn_lm" in conf.arch
    logger, timer = run.logger, run.timer
    tracker_tr = RuntimeTracker(metrics.metric_names, on_cuda=graph.on_cuda, world_aggregator=optimizer.world_aggregator)
    pending = _PendingRecords()
    rank_slice = slice(graph.rank * conf.batch_size, (graph.rank + 1) * conf.batch_size) if is_nlp else None
    step_fn, hidden = None, None
    step_cache = {}   # one TrainStep (one captured graph) per batch shape, reused across epochs
    elastic = _Elastic(conf, run) if run.membership is not None else None
    global_rank = dist.get_rank() if (dist.is_available() and dist.is_initialized()) else 0
    print("=> enter the training.\n")
    while True:
        _barrier(run.group)
        for _input, _target in data_loader["train_loader"]:
            if elastic is not None:
                if elastic.wants_to_leave(global_rank, scheduler.local_index + 1):
                    elastic.leave(optimizer)
                    logger.save_json()
                    run.extras["lost_ranks"] = [global_rank]
                    return scheduler
                seen = elastic.lost_now(optimizer, scheduler.local_index + 1)
                if seen:
                    pending.flush(logger, graph, tracker_tr, metrics.metric_names, False)
                    graph, optimizer = elastic.recover(seen, graph, model, optimizer, scheduler)
                    tracker_tr = RuntimeTracker(metrics.metric_names, on_cuda=graph.on_cuda,
                                                world_aggregator=optimizer.world_aggregator)
                    step_fn, step_cache = None, {}
                    break   # all survivors restart the pass over their loaders together
            model.train()
            scheduler.step(optimizer)
            with timer("load_data", epoch=scheduler.epoch_):
                if is_nlp:
                    _input, _target = _input[:, rank_slice], _target[:, rank_slice]
                    if _input.size(0) != conf.rnn_bptt_len or _input.size(1) != conf.batch_size:
                        continue  # ragged tail window
                shape_key = tuple(_input.shape)
                if step_fn is None or tuple(step_fn.static_input.shape) != shape_key:
                    step_fn = step_cache.get(shape_key)
                if step_fn is None:
                    if is_nlp:
                        hidden = tuple(h.to(optimizer.device) for h in model.init_hidden(conf.batch_size))
                    step_fn = step_cache[shape_key] = TrainStep(
                        model, criterion, optimizer, _input, _target, metrics=metrics,
                        use_cuda_graph=conf.use_cuda_graph and _input.size(0) == (conf.rnn_bptt_len if is_nlp else conf.batch_size),
                        clip_grad_norm=conf.rnn_clip if is_nlp else None, hidden=hidden,
                        amp_dtype=torch.bfloat16 if conf.dtype == "bf16" else None,
                        gossip_bucket_mb=getattr(conf, "gossip_bucket_mb", 0.0),
                    )
            try:
                with timer("forward_pass", epoch=scheduler.epoch_):
                    loss = step_fn(_input, _target, timer=timer, scheduler=scheduler)
            except RuntimeError as e:
                # a rank left between this rank's membership check and its exchange: the send / receive (or
                # the bounded device wait) fails instead of hanging; continue on the survivors
                if elastic is None:
                    raise
                seen = elastic.after_failure(e)
                pending.flush(logger, graph, tracker_tr, metrics.metric_names, False)
                graph, optimizer = elastic.recover(seen, graph, model, optimizer, scheduler)
                tracker_tr = RuntimeTracker(metrics.metric_names, on_cuda=graph.on_cuda,
                                            world_aggregator=optimizer.world_aggregator)
                step_fn, step_cache = None, {}
                break
            n_bits = optimizer.n_bits
            pending.add({"n": _input.size(1) if is_nlp else _input.size(0), "bits": n_bits, "sched": _SchedView(scheduler)},
                        loss, step_fn.perf)
            if scheduler.local_index % conf.summary_freq == 0 or scheduler.epoch_ % 1 == 0 or scheduler.is_stop():
                pending.flush(logger, graph, tracker_tr, metrics.metric_names, False)
                if elastic is None:
                    optimizer.check()   # a bounded device-side wait that ran out ends the run here
            if scheduler.epoch_ % 1 == 0 or scheduler.is_stop():
                avg = tracker_tr.stat["loss"].avg
                if avg > 1e3 or math.isnan(avg):
                    logger.save_json()
                    raise TrainingDiverged(f"loss average {avg} at epoch {scheduler.epoch_}")
                do_validate(conf, graph, run, model, optimizer, criterion, scheduler, metrics, data_loader, device,
                            rank_slice)
                tracker_tr.reset()
                if (conf.evaluate_consensus or scheduler.is_stop()) and not conf.train_fast and not is_nlp:
                    consensus_evaluation(conf, graph, run, model, optimizer, criterion, scheduler, metrics, device)
                if scheduler.is_stop():
                    logger.save_json()
                    optimizer.finalize()
                    return scheduler
            if graph.rank == 0 and conf.display_tracked_time and scheduler.local_index % conf.summary_freq == 0:
                print(timer.summary())
        if conf.reshuffle_per_epoch:
            print("\nReshuffle the dataset.")
            del data_loader
            gc.collect()
            data_loader = define_dataset(conf, graph, run, device=device)


def consensus_evaluation(conf, graph, run, model, optimizer, criterion, scheduler, metrics, device):
    """Evaluate the local and the world-averaged model on the whole (unpartitioned) training set
    (``dl_code/pcode/distributed_running_cv.py:81-126``)."""
    full = conf.replace(partition_data=None)
    from ..config import RunState

    loaders = define_dataset(full, graph, RunState())
    dl = {"val_loader": loaders["train_loader"]}
    run.logger.log("eval the local model on full training data.")
    validate(conf, graph, run, model, optimizer, criterion, scheduler, metrics, dl,
             label="eval_local_model_on_full_training_data", force_evaluate_on_averaged_model=False, device=device)
    run.logger.log("eval the averaged model on full training data.")
    copied = copy.deepcopy(model)
    optimizer.world_aggregator.agg_model(copied, op="avg")
    validate(conf, graph, run, copied, optimizer, criterion, scheduler, metrics, dl,
             label="eval_averaged_model_on_full_training_data", force_evaluate_on_averaged_model=False, device=device)
