"""Curve plotting versus step / epoch / time with smoothing and grouping
(``dl_code/pcode/tools/plot.py:14-153``, ``plot_utils.py:11-219``).  matplotlib is imported
on use; without it ``plot_curves`` writes the same series as CSV next to the requested file."""
from __future__ import annotations

import csv
from typing import Dict, Sequence, Tuple


def smooth(ys: Sequence[float], window: int = 1):
    if window <= 1:
        return list(ys)
    out, acc = [], 0.0
    for i, y in enumerate(ys):
        acc += y
        if i >= window:
            acc -= ys[i - window]
        out.append(acc / min(i + 1, window))
    return out


def group_mean(curves: Sequence[Tuple[Sequence[float], Sequence[float]]]):
    """Mean and std over repetitions at shared x."""
    acc = {}
    for xs, ys in curves:
        for x, y in zip(xs, ys):
            acc.setdefault(x, []).append(y)
    xs = sorted(acc)
    mean = [sum(acc[x]) / len(acc[x]) for x in xs]
    std = [(sum((v - m) ** 2 for v in acc[x]) / len(acc[x])) ** 0.5 for x, m in zip(xs, mean)]
    return xs, mean, std


def plot_curves(series: Dict[str, Tuple[Sequence[float], Sequence[float]]], path: str, xlabel="epoch", ylabel="",
                logy=False, window=1, title=None):
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        csv_path = path.rsplit(".", 1)[0] + ".csv"
        with open(csv_path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["label", xlabel, ylabel or "value"])
            for label, (xs, ys) in series.items():
                for x, y in zip(xs, smooth(ys, window)):
                    w.writerow([label, x, y])
        return csv_path
    fig, ax = plt.subplots(figsize=(6, 4))
    for label, (xs, ys) in series.items():
        ax.plot(xs, smooth(ys, window), label=label)
    ax.set_xlabel(xlabel)
    ax.set_ylabel(ylabel)
    if logy:
        ax.set_yscale("log")
    if title:
        ax.set_title(title)
    ax.legend()
    fig.tight_layout()
    fig.savefig(path)
    plt.close(fig)
    return path
