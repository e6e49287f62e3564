"""Learning-rate schedule evaluated at fractional epochs, plus training progress.

Behaviour of ``dl_code/pcode/create_scheduler.py:6-403``:

* base LR: ``lr / base_batch_size * batch_size``, scaled by the neighbourhood size
  (``graph``), the world size, an explicit factor, or the ``sqrt`` rule;
* schemes: ``strict`` (explicit epoch fields / LR fields / interpolation kinds),
  ``custom_one_cycle``, ``custom_multistep`` (optional linear warm-up from ``lr`` to the
  scaled LR, then division by ``lr_decay`` at every change epoch),
  ``custom_convex_decay`` (gamma / (mu (t + alpha)));
* ``step()`` advances ``local_index``, recomputes ``epoch_ = local_index / batches_per_epoch``
  and writes the new LR into every param group when it changed.

A schedule is a list of ``Piece(epoch_left, epoch_right, fn)``; the reference builds the
same thing out of three comma/slash separated strings."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

from ..utils.auxiliary import is_float


@dataclass
class Piece:
    left: float
    right: float
    fn: Callable[[float], float]
    kind: str
    lr_left: float
    lr_right: float


def linear_piece(l, r, lr_l, lr_r):
    n = r - l
    return Piece(l, r, lambda e: (e - l) * ((lr_r - lr_l) / n) + lr_l, "linear", lr_l, lr_r)


def poly_piece(l, r, lr_l, lr_r):
    n = r - l
    return Piece(l, r, lambda e: lr_l * ((1 - (e - l) / n) ** 2), "poly", lr_l, lr_r)


def convex_piece(l, r, gamma, mu, alpha):
    return Piece(l, r, lambda e: gamma / (mu * (alpha + e)), "convex", gamma / (mu * (alpha + l)), 0.0)


_KINDS = {"0": "linear", "1": "poly", "2": "convex"}


def scaled_learning_rate(conf, graph) -> float:
    base_bs = conf.base_batch_size if conf.base_batch_size is not None else conf.batch_size
    per_sample = conf.lr / base_bs
    if not conf.lr_scaleup:
        return per_sample * conf.batch_size
    if conf.lr_scaleup_type == "linear":
        lr = per_sample * conf.batch_size
        if is_float(conf.lr_scaleup_factor):
            scale = float(conf.lr_scaleup_factor)
        elif conf.lr_scaleup_factor == "graph":
            scale = graph.scaling
        elif conf.lr_scaleup_factor == "world":
            scale = graph.n_nodes
        else:
            raise NotImplementedError(conf.lr_scaleup_factor)
    elif conf.lr_scaleup_type == "sqrt":
        lr = conf.lr
        scale = (1.0 * graph.n_nodes * conf.batch_size / base_bs) ** 0.5
    else:
        raise NotImplementedError(conf.lr_scaleup_type)
    return lr * scale


def build_pieces(conf, learning_rate: float, init_warmup_lr: float) -> Optional[List[Piece]]:
    scheme = conf.lr_schedule_scheme
    if scheme is None or scheme == "reduce_on_plateau":
        return None
    if scheme == "strict":
        epochs = [0] + [int(e) for e in conf.lr_change_epochs.split(",")] + [conf.num_epochs]
        fields = [[float(v) for v in f.split(",")] for f in conf.lr_fields.split("/")]
        kinds = [_KINDS[k] for k in conf.lr_scale_indicators.split(",")]
    elif scheme == "custom_one_cycle":
        low, high, xlow = conf.lr_onecycle_low, conf.lr_onecycle_high, conf.lr_onecycle_extra_low
        epochs = [0, conf.lr_onecycle_num_epoch // 2, conf.lr_onecycle_num_epoch, conf.num_epochs]
        fields = [[low, high], [high, low], [low, xlow]]
        kinds = ["linear"] * 3
    elif scheme == "custom_multistep":
        changes = [int(e) for e in conf.lr_change_epochs.split(",")] if conf.lr_change_epochs else []
        levels = [learning_rate * ((1.0 / conf.lr_decay) ** l) for l in range(len(changes) + 1)]
        fields = [[lr, lr] for lr in levels]
        epochs = [0] + changes + [conf.num_epochs]
        if conf.lr_warmup:
            fields = [[init_warmup_lr, learning_rate]] + fields
            epochs = [0, conf.lr_warmup_epochs] + epochs[1:]
        kinds = ["linear"] * (len(epochs) - 1)
    elif scheme == "custom_convex_decay":
        epochs = [0, conf.num_epochs]
        fields = [[learning_rate, 0.0]]
        kinds = ["convex"]
    else:
        raise NotImplementedError(scheme)
    pieces = []
    for (l, r), (lr_l, lr_r), kind in zip(zip(epochs[:-1], epochs[1:]), fields, kinds):
        if kind == "linear":
            pieces.append(linear_piece(l, r, lr_l, lr_r))
        elif kind == "poly":
            pieces.append(poly_piece(l, r, lr_l, lr_r))
        else:
            assert conf.lr_gamma is not None and conf.lr_mu is not None and conf.lr_alpha is not None
            pieces.append(convex_piece(l, r, conf.lr_gamma, conf.lr_mu, conf.lr_alpha))
    return pieces


class Scheduler:
    def __init__(self, conf, graph, run):
        self.conf, self.graph, self.run = conf, graph, run
        self.local_index = run.local_index
        self.epoch_ = 0.0
        self.epoch = 0
        self.best_tracker = None
        run.init_warmup_lr = conf.lr
        run.learning_rate = scaled_learning_rate(conf, graph)
        self.learning_rate = run.learning_rate
        self.old_learning_rate = run.learning_rate
        self.pieces = build_pieces(conf, run.learning_rate, run.init_warmup_lr)

    def update_from_checkpoint(self, checkpoint):
        self.local_index = self.run.local_index = checkpoint["local_index"]
        self.run.best_perf = checkpoint["best_perf"]

    def set_best_tracker(self, best_tracker):
        self.best_tracker = best_tracker

    def state_dict(self):
        return {"local_index": self.local_index, "epoch_": self.epoch_, "old_learning_rate": self.old_learning_rate}

    def load_state_dict(self, sd):
        self.local_index = sd["local_index"]
        self.epoch_ = sd.get("epoch_", 0.0)
        self.old_learning_rate = sd.get("old_learning_rate", self.old_learning_rate)

    def get_lr(self, epoch_=None):
        e = self.epoch_ if epoch_ is None else epoch_
        if self.pieces is None:
            return None
        for p in self.pieces:
            if p.left <= e < p.right:
                return p.fn(e)
        return None

    def step(self, optimizer=None, **_):
        self.update_training_progress()
        lr = self.get_lr()
        if lr is None:
            lr = self.old_learning_rate
        if optimizer is not None and (self.old_learning_rate != lr or self.local_index == 1):
            for g in optimizer.param_groups:
                g["lr"] = lr
        self.old_learning_rate = lr
        return lr

    def update_training_progress(self):
        self.local_index += 1
        self.epoch_ = self.local_index / self.run.num_batches_train_per_device_per_epoch
        self.epoch = int(self.epoch_)
        self.run.local_index, self.run.epoch_, self.run.epoch = self.local_index, self.epoch_, self.epoch

    def is_stop(self):
        if self.conf.steps is not None and self.local_index >= self.conf.steps:
            return True
        if self.conf.stop_criteria == "epoch":
            return self.epoch >= self.conf.num_epochs
        if self.conf.stop_criteria == "iteration":
            return self.local_index >= self.run.num_iterations_per_worker
        raise NotImplementedError(self.conf.stop_criteria)
