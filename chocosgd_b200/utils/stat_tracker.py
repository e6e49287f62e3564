"""Running statistics (``dl_code/pcode/utils/stat_tracker.py:7-133``).

``RuntimeTracker`` additionally accepts 0-d device tensors: sums stay on the device and are
only read back when a record is written, so the training loop has no per-step host sync
(the reference calls ``.item()`` on loss and on every accuracy each step)."""
from __future__ import annotations

from copy import deepcopy

import torch


class MaxMeter:
    def __init__(self):
        self.max = None

    def update(self, value):
        if self.max is None or value > self.max:
            self.max = deepcopy(value)
            return True
        return False

    def value(self):
        return self.max


class MinMeter:
    def __init__(self):
        self.min = None

    def update(self, value):
        if self.min is None or value < self.min:
            self.min = deepcopy(value)
            return True
        return False

    def value(self):
        return self.min


def _f(v):
    return float(v.item()) if torch.is_tensor(v) else float(v)


class AverageMeter:
    def __init__(self):
        self.reset()

    def reset(self):
        self.val = 0
        self.sum = 0
        self.count = 0
        self.max = -float("inf")
        self.min = float("inf")

    def update(self, val, n=1):
        self.val = val
        self.sum = self.sum + val * n
        self.count += n
        if not torch.is_tensor(val):
            self.max = max(self.max, val)
            self.min = min(self.min, val)

    @property
    def avg(self):
        return _f(self.sum) / max(self.count, 1)


class RuntimeTracker:
    def __init__(self, metrics_to_track=("top1",), on_cuda=True, world_aggregator=None):
        self.metrics_to_track = list(metrics_to_track)
        self.things_to_track = ["loss"] + self.metrics_to_track
        self.on_cuda = on_cuda
        self.world_aggregator = world_aggregator
        self.reset()

    def reset(self):
        self.stat = {name: AverageMeter() for name in self.things_to_track}

    def evaluate_global_metric(self, metric):
        s, c = _f(self.stat[metric].sum), float(self.stat[metric].count)
        if self.world_aggregator is None:
            return s / max(c, 1.0)
        return self.world_aggregator.global_average(s, c)

    def evaluate_global_metrics(self):
        return [self.evaluate_global_metric(m) for m in self.metrics_to_track]

    def get_metrics_performance(self):
        return [self.stat[m].avg for m in self.metrics_to_track]

    def update_metrics(self, metric_stat, n_samples):
        for idx, thing in enumerate(self.things_to_track):
            self.stat[thing].update(metric_stat[idx], n_samples)

    def __call__(self):
        return {name: val.avg for name, val in self.stat.items()}


class BestPerf:
    def __init__(self, best_perf=None, larger_is_better=True):
        self.best_perf = best_perf
        self.cur_perf = None
        self.best_perf_locs = []
        self.larger_is_better = larger_is_better
        self.is_best = False
        self.meter = MaxMeter() if larger_is_better else MinMeter()
        if best_perf is not None:
            self.meter.update(best_perf)

    def update(self, perf, perf_location):
        self.is_best = self.meter.update(perf)
        self.cur_perf = perf
        if self.is_best:
            self.best_perf = perf
            self.best_perf_locs += [perf_location]

    def get_best_perf_loc(self):
        return self.best_perf_locs[-1] if self.best_perf_locs else None
