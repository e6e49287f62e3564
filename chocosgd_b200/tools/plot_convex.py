"""Sub-optimality curves of the convex experiments: f(x_bar) - f* versus epoch and versus the
number of transmitted bits (``convex_code/plots-epsilon.ipynb:39,89-95,195-309``).

    python -m chocosgd_b200.tools.plot_convex <experiment dir> --baseline baselines.pickle --out plots/

``<experiment dir>`` holds ``params.pickle`` and ``results.pickle`` written by
``convex/experiment.py``.  Curves of runs that differ only in the seed are averaged (mean, with a
min / max band).  The bits axis uses the per-node, per-iteration model of the reference's plots:
full 64 * 2 * d, random-k 64 * 2 * k, top-k (64 + ceil(log2 d)) * 2 * k, QSGD
(ceil(log2 levels) + 1) * 2 * d."""
from __future__ import annotations

import argparse
import os
import pickle
import re
from typing import Dict, List, Tuple

import numpy as np

from ..convex.logistic import LOSS_PER_EPOCH, LogisticDecentralizedSGD
from .plot import plot_curves


def bits_per_node_iteration(param, d: int) -> float:
    return float(LogisticDecentralizedSGD(param).bits_per_node_iteration(d))


def _group_name(param) -> str:
    name = str(param)
    return re.sub(r"-seed\d+$", "", name)


def suboptimality_curves(params, results, f_star: float, n_samples: int, d: int):
    """{group: {"epoch": xs, "bits": xs, "mean": ys, "lo": ys, "hi": ys}} from the 10-per-epoch loss traces."""
    groups: Dict[str, List[Tuple[object, np.ndarray]]] = {}
    for p, (_, trace) in zip(params, results):
        groups.setdefault(_group_name(p), []).append((p, np.asarray(trace, dtype=np.float64)))
    out = {}
    for g, runs in groups.items():
        p0 = runs[0][0]
        n = min(len(t) for _, t in runs)
        sub = np.stack([t[:n] for _, t in runs]) - f_star
        per_node = n_samples // p0.n_cores if p0.distribute_data else n_samples
        every = max(1, int(per_node / LOSS_PER_EPOCH))
        iters = np.arange(n) * every
        out[g] = {
            "epoch": iters / per_node,
            "bits": iters * p0.n_cores * bits_per_node_iteration(p0, d),
            "mean": sub.mean(axis=0), "lo": sub.min(axis=0), "hi": sub.max(axis=0),
            "n_runs": len(runs),
        }
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("directory")
    ap.add_argument("--baseline", default=None, help="pickle with the optimal loss f* (default: 0)")
    ap.add_argument("--n_samples", type=int, default=None)
    ap.add_argument("--n_features", type=int, default=None)
    ap.add_argument("--out", default=".")
    a = ap.parse_args(argv)
    with open(os.path.join(a.directory, "params.pickle"), "rb") as f:
        params = pickle.load(f)
    with open(os.path.join(a.directory, "results.pickle"), "rb") as f:
        results = pickle.load(f)
    f_star = 0.0
    if a.baseline:
        with open(a.baseline, "rb") as f:
            f_star = float(pickle.load(f))
    n = a.n_samples or int(round(1.0 / params[0].regularizer))
    d = a.n_features or int(params[0].tau)
    curves = suboptimality_curves(params, results, f_star, n, d)
    os.makedirs(a.out, exist_ok=True)
    written = []
    for axis, xlabel in (("epoch", "epoch"), ("bits", "transmitted bits")):
        series = {g: (c[axis][1:], np.maximum(c["mean"][1:], 1e-16)) for g, c in curves.items()}
        bands = {g: (np.maximum(c["lo"][1:], 1e-16), np.maximum(c["hi"][1:], 1e-16)) for g, c in curves.items()}
        written.append(plot_curves(series, os.path.join(a.out, f"suboptimality_vs_{axis}.png"), xlabel=xlabel,
                                   ylabel="f(x) - f*", logy=True, logx=(axis == "bits"), bands=bands))
    print("\n".join(written))
    return curves


if __name__ == "__main__":
    main()
