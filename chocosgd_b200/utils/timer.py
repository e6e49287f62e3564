"""Scoped timer with CUDA-event timing.

Same interface as the reference (``with timer(label, epoch=...)``, ``summary()``,
first occurrence skipped, sampled logging with probability 1/count;
``dl_code/pcode/utils/timer.py:10-120``) but GPU scopes are bracketed by CUDA events
recorded on the current stream instead of ``torch.cuda.synchronize()`` on both sides of
every scope, which would serialise the gossip/compute overlap.  Event pairs are resolved
lazily (``flush``) once they have completed.  Optional NVTX ranges carry the same labels.
"""
from __future__ import annotations

import time
from contextlib import contextmanager
from io import StringIO

import numpy as np
import torch


class Timer:
    def __init__(self, verbosity_level=1, log_fn=None, skip_first=True, on_cuda=True, nvtx=False):
        self.verbosity_level = verbosity_level
        self.log_fn = log_fn if log_fn is not None else self._default_log_fn
        self.skip_first = skip_first
        self.cuda_available = torch.cuda.is_available() and on_cuda
        self.nvtx = nvtx and self.cuda_available
        self._rng = np.random.RandomState(0)
        self.reset()

    def reset(self):
        self.totals = {}
        self.first_time = {}
        self.last_time = {}
        self.call_counts = {}
        self._pending = []  # (label, epoch, start_event, end_event, wall_start, wall_end)

    @contextmanager
    def __call__(self, label, epoch=-1.0, verbosity=1):
        if verbosity > self.verbosity_level:
            yield
            return
        if self.nvtx:
            torch.cuda.nvtx.range_push(label)
        if self.cuda_available:
            ev0 = torch.cuda.Event(enable_timing=True)
            ev1 = torch.cuda.Event(enable_timing=True)
            ev0.record()
        start = time.time()
        yield
        end = time.time()
        if self.cuda_available:
            ev1.record()
            self._pending.append((label, epoch, ev0, ev1, start, end))
            if len(self._pending) > 256:
                self.flush(block=False)
        else:
            self._account(label, epoch, end - start, start, end)
        if self.nvtx:
            torch.cuda.nvtx.range_pop()

    def flush(self, block=True):
        """Resolve finished event pairs into the totals."""
        keep = []
        for rec in self._pending:
            label, epoch, ev0, ev1, start, end = rec
            if block:
                ev1.synchronize()
            if ev1.query():
                self._account(label, epoch, ev0.elapsed_time(ev1) * 1e-3, start, end)
            else:
                keep.append(rec)
        self._pending = keep

    def _account(self, label, epoch, duration, start, end):
        if label not in self.first_time:
            self.first_time[label] = start
        self.last_time[label] = end
        if label not in self.totals and self.skip_first:
            self.totals[label] = 0.0
            del self.first_time[label]
            self.call_counts[label] = 0
        elif label not in self.totals:
            self.totals[label] = duration
            self.call_counts[label] = 1
        else:
            self.totals[label] += duration
            self.call_counts[label] += 1
        if self.call_counts[label] > 0 and self._rng.rand() < 1 / self.call_counts[label]:
            self.log_fn("timer", {"epoch": epoch, "value": duration}, {"event": label})

    def summary(self):
        self.flush()
        if not self.totals:
            return ""
        with StringIO() as buf:
            total_avg, count = 0.0, 0
            print("--- Timer summary ------------------------", file=buf)
            print("  Event   |  Count | Average time |  Frac.", file=buf)
            for label in sorted(self.totals):
                total, count = self.totals[label], self.call_counts[label]
                if count == 0:
                    continue
                avg = total / count
                runtime = max(self.last_time[label] - self.first_time.get(label, self.last_time[label]), 1e-12)
                total_avg += avg if "." not in label else 0  # dotted labels are sub-events
                print(f"- {label:30s} | {count:6d} | {avg:11.5f}s | {100 * total / runtime:5.1f}%", file=buf)
            print("-------------------------------------------", file=buf)
            print(f"- {'total_averaged_time':30s}| {count:6d} | {total_avg:11.5f}s |", file=buf)
            print("-------------------------------------------", file=buf)
            return buf.getvalue()

    def _default_log_fn(self, _, values, tags):
        print(f"Timer: {tags['event']:30s} @ {values['epoch']:4.1f} - {values['value']:8.5f}s")
