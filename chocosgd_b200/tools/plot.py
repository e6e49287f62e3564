"""Curves of finished runs: any logged metric versus step, epoch, wall-clock time or transmitted
bits; trailing-window smoothing, sub-ranges, log axes, one legend entry per configuration,
repetitions averaged with a band, and the accuracy-versus-global-batch scatter
(``dl_code/pcode/tools/plot.py:14-153``, ``dl_code/pcode/tools/plot_utils.py:11-219``).

    python -m chocosgd_b200.tools.plot <checkpoint root> --split test_local --metric top1 --x epoch \
        --legend optimizer,comm_op,graph_topology --out top1.png

matplotlib is imported on use; where it is missing every function writes the series it would have
drawn as CSV next to the requested file and returns that path."""
from __future__ import annotations

import argparse
import csv
import datetime
from itertools import groupby
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

LINE_STYLES = ["-", "--", "-.", ":"]
COLORS = ["#377eb8", "#ff7f00", "#4daf4a", "#f781bf", "#a65628", "#984ea3", "#999999", "#e41a1c", "#dede00"]
MARKERS = ["o", "v", "^", "<", ">", "8", "s", "p", "*", "h", "H", "D", "d", "P", "X"]


# ---- operations on (x, y) -------------------------------------------------------------------------------
def smooth(ys: Sequence[float], window: int = 1) -> List[float]:
    """Mean over the ``window`` values that precede each point (the point itself when none do)."""
    if window <= 1:
        return list(ys)
    out, acc = [], 0.0
    for i, y in enumerate(ys):
        acc += y
        if i >= window:
            acc -= ys[i - window]
        out.append(acc / min(i + 1, window))
    return out


def smoothing_func(x, y, smooth_length=10):
    return list(x), smooth(list(y), smooth_length)


def reject_outliers(data, threshold=3.0):
    import numpy as np

    data = np.asarray(data, dtype=float)
    return data[abs(data - data.mean()) < threshold * data.std()]


def subset(xs, ys, left=0.0, right=1.0):
    a, b = int(len(xs) * left), int(len(xs) * right)
    return list(xs[a:b]), list(ys[a:b])


def drop_first_few(xs, ys, num_drop):
    return list(xs[num_drop:]), list(ys[num_drop:])


def sample_from_records(xs, ys, local_step=1, max_same_num_sync=None):
    """Every ``local_step``-th record (one per synchronisation), cut to a common number of syncs."""
    if max_same_num_sync is not None:
        xs, ys = xs[: local_step * max_same_num_sync], ys[: local_step * max_same_num_sync]
    return list(xs[::local_step]), list(ys[::local_step])


def find_same_num_sync(steps_and_local_steps: Iterable[Tuple[int, int]]) -> int:
    return min(n // k for n, k in steps_and_local_steps)


def seconds_since_start(times: Sequence) -> List[float]:
    """Wall-clock x axis from record time stamps (datetime objects, ISO strings or seconds)."""
    def as_seconds(t):
        if isinstance(t, (int, float)):
            return float(t)
        if isinstance(t, str):
            for fmt in ("%Y-%m-%d %H:%M:%S", "%Y-%m-%dT%H:%M:%S", "%Y-%m-%d %H:%M:%S.%f"):
                try:
                    return datetime.datetime.strptime(t, fmt).timestamp()
                except ValueError:
                    continue
            return float(t)
        return t.timestamp()

    secs = [as_seconds(t) for t in times]
    return [s - secs[0] + 1 for s in secs]


def add_communication_delay(times, local_step, delay_factor):
    return [t + delay_factor * ((i + 1) // local_step) for i, t in enumerate(times)]


def group_mean(curves: Sequence[Tuple[Sequence[float], Sequence[float]]]):
    """Mean and standard deviation over repetitions at shared x."""
    acc = {}
    for xs, ys in curves:
        for x, y in zip(xs, ys):
            acc.setdefault(x, []).append(y)
    xs = sorted(acc)
    mean = [sum(acc[x]) / len(acc[x]) for x in xs]
    std = [(sum((v - m) ** 2 for v in acc[x]) / len(acc[x])) ** 0.5 for x, m in zip(xs, mean)]
    return xs, mean, std


# ---- grouping and legends --------------------------------------------------------------------------------
def groupby_indices(results, grouper):
    return [(k, list(g)) for k, g in groupby(sorted(results, key=grouper), grouper)]


def build_legend(arguments: dict, legend: str) -> str:
    """``"optimizer,lr"`` -> ``"optimizer=sgd, lr=0.1"``."""
    return ", ".join("{}={}".format(k, arguments.get(k)) for k in legend.split(",") if k)


def determine_color_and_lines(ind: int, n_cases: Optional[int] = None):
    """(line style, colour, marker) of the ``ind``-th curve: colours cycle first, then line styles."""
    return LINE_STYLES[(ind // len(COLORS)) % len(LINE_STYLES)], COLORS[ind % len(COLORS)], MARKERS[ind % len(MARKERS)]


def reorder_records(exps, based_on: str):
    return sorted(exps, key=lambda e: str(e["arguments"].get(based_on)))


# ---- series from experiment records -----------------------------------------------------------------------
def series_of(exp, split="train", metric="loss", x="epoch"):
    """(xs, ys) of one experiment.  ``x`` in {"step", "epoch", "time", "bits"}: bits is the running
    sum of the logged ``n_bits_to_transmit`` (MB per step) of rank 0."""
    from .show_results import curve, split_records

    if x in ("epoch", "local_index"):
        return curve(exp, split, metric, x)
    ranks = sorted(exp["records"])
    if not ranks:
        return [], []
    recs = [r for r in split_records(exp["records"][ranks[0]])[split] if metric in r]
    ys = [float(r[metric]) for r in recs]
    if x == "step":
        return [float(r.get("local_index", i + 1)) for i, r in enumerate(recs)], ys
    if x == "time":
        return seconds_since_start([r["time"] for r in recs]), ys
    if x == "bits":
        total, xs = 0.0, []
        for r in recs:
            total += float(r.get("n_bits_to_transmit", 0.0))
            xs.append(total)
        return xs, ys
    raise ValueError(x)


def collect_series(exps, legend="optimizer,comm_op", split="test_local", metric="top1", x="epoch", window=1,
                   left=0.0, right=1.0, reorder_by=None):
    """One series per distinct legend string; experiments that share it are averaged (mean, std band)."""
    if reorder_by:
        exps = reorder_records(exps, reorder_by)
    grouped: Dict[str, list] = {}
    for e in exps:
        xs, ys = series_of(e, split, metric, x)
        if ys:
            grouped.setdefault(build_legend(e["arguments"], legend), []).append((xs, ys))
    series, bands = {}, {}
    for label, curves in grouped.items():
        xs, mean, std = group_mean(curves) if len(curves) > 1 else (curves[0][0], curves[0][1], None)
        ys = smooth(mean, window)
        series[label] = subset(xs, ys, left, right)
        if std is not None:
            lo, hi = [m - s for m, s in zip(ys, std)], [m + s for m, s in zip(ys, std)]
            bands[label] = (subset(xs, lo, left, right)[1], subset(xs, hi, left, right)[1])
    return series, bands


# ---- drawing ---------------------------------------------------------------------------------------------------
def _pyplot():
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt

        return plt
    except ImportError:
        return None


def _write_csv(series, path, xlabel, ylabel, bands=None):
    csv_path = path.rsplit(".", 1)[0] + ".csv"
    with open(csv_path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["label", xlabel, ylabel or "value", "low", "high"])
        for label, (xs, ys) in series.items():
            lo, hi = (bands or {}).get(label, (None, None))
            for i, (x, y) in enumerate(zip(xs, ys)):
                w.writerow([label, x, y, "" if lo is None else lo[i], "" if hi is None else hi[i]])
    return csv_path


def configure_figure(ax, xlabel, ylabel, title=None, has_legend=True, legend_loc="best", legend_ncol=1,
                     bbox_to_anchor=None):
    if has_legend:
        kw = dict(loc=legend_loc, ncol=legend_ncol, shadow=True, fancybox=True, fontsize=9)
        if bbox_to_anchor is not None:
            kw["bbox_to_anchor"] = bbox_to_anchor
        ax.legend(**kw)
    ax.set_xlabel(xlabel)
    ax.set_ylabel(ylabel)
    if title:
        ax.set_title(title)
    return ax


def plot_curves(series: Dict[str, Tuple[Sequence[float], Sequence[float]]], path: str, xlabel="epoch", ylabel="",
                logy=False, logx=False, window=1, title=None, bands=None, mark_every=None, ylim=(None, None),
                legend_loc="best", legend_ncol=1):
    series = {k: (list(xs), smooth(list(ys), window)) for k, (xs, ys) in series.items()}
    plt = _pyplot()
    if plt is None:
        return _write_csv(series, path, xlabel, ylabel, bands)
    fig, ax = plt.subplots(figsize=(7, 4.5))
    for i, (label, (xs, ys)) in enumerate(series.items()):
        ls, color, marker = determine_color_and_lines(i, len(series))
        ax.plot(xs, ys, label=label, linestyle=ls, color=color, linewidth=1.8,
                marker=marker if mark_every else None, markevery=mark_every)
        if bands and label in bands:
            ax.fill_between(xs, bands[label][0], bands[label][1], color=color, alpha=0.15, linewidth=0)
    if logy:
        ax.set_yscale("log")
    if logx:
        ax.set_xscale("log")
    ax.set_ylim(bottom=ylim[0], top=ylim[1])
    configure_figure(ax, xlabel, ylabel, title, legend_loc=legend_loc, legend_ncol=legend_ncol)
    fig.tight_layout()
    fig.savefig(path)
    plt.close(fig)
    return path


def plot_curve_wrt(exps, path, x="epoch", split="test_local", metric="top1", legend="optimizer,comm_op", **kw):
    """The reference's ``plot_curve_wrt_time`` generalised to any x axis."""
    plot_kw = {k: kw.pop(k) for k in list(kw) if k in ("logy", "logx", "title", "mark_every", "ylim", "legend_loc",
                                                       "legend_ncol")}
    series, bands = collect_series(exps, legend, split, metric, x, **kw)
    xlabel = {"epoch": "epoch", "step": "step", "local_index": "step", "time": "seconds", "bits": "transmitted MB"}[x]
    return plot_curves(series, path, xlabel=xlabel, ylabel=metric, bands=bands, **plot_kw)


def best_by_global_minibatch_size(exps, metric="top1", split="test_local"):
    """[(lr, [(global batch, best metric), ...])]: the best run per (nodes, lr, global batch)."""
    rows = []
    for e in exps:
        a = e["arguments"]
        _, ys = series_of(e, split, metric, "epoch")
        if ys:
            n = int(a.get("n_mpi_process", a.get("n_nodes", 1)))
            rows.append((n, a.get("lr"), int(a.get("batch_size", 0)) * n, max(ys)))
    best = [max(g, key=lambda r: r[-1]) for _, g in groupby_indices(rows, lambda r: (r[0], str(r[1]), r[2]))]
    return [(lr, sorted((r[2], r[3]) for r in g)) for lr, g in groupby_indices(best, lambda r: str(r[1]))]


def plot_by_global_minibatch_size(exps, path, metric="top1", split="test_local"):
    groups = best_by_global_minibatch_size(exps, metric, split)
    series = {"lr={}".format(lr): ([p[0] for p in pts], [p[1] for p in pts]) for lr, pts in groups}
    plt = _pyplot()
    if plt is None:
        return _write_csv(series, path, "global batch size", metric)
    fig, ax = plt.subplots(figsize=(7, 4.5))
    ticks = set()
    for i, (label, (xs, ys)) in enumerate(series.items()):
        _, color, marker = determine_color_and_lines(i)
        ax.scatter(xs, ys, c=color, marker=marker, s=60, label=label)
        ticks.update(xs)
    ax.set_xscale("log", base=2)
    ax.set_xticks(sorted(ticks))
    ax.set_xticklabels(sorted(ticks))
    configure_figure(ax, "global batch size", metric)
    fig.tight_layout()
    fig.savefig(path)
    plt.close(fig)
    return path


def main(argv=None):
    from .show_results import find_experiments

    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("root")
    p.add_argument("--split", default="test_local", choices=("train", "test_local", "test_averaged", "test_best"))
    p.add_argument("--metric", default="top1")
    p.add_argument("--x", default="epoch", choices=("epoch", "step", "time", "bits"))
    p.add_argument("--legend", default="optimizer,comm_op,graph_topology")
    p.add_argument("--where", default="", help="k=v,k=v filter on the run arguments")
    p.add_argument("--smooth", type=int, default=1)
    p.add_argument("--logy", action="store_true")
    p.add_argument("--out", default="curves.png")
    a = p.parse_args(argv)
    cond = dict(kv.split("=", 1) for kv in a.where.split(",") if kv)
    exps = find_experiments(a.root, cond)
    print(plot_curve_wrt(exps, a.out, x=a.x, split=a.split, metric=a.metric, legend=a.legend, window=a.smooth,
                         logy=a.logy))


if __name__ == "__main__":
    main()
