"""Sweep driver: run a list of parameter sets in a process pool and pickle the results
(``convex_code/experiment.py:16-40``); ``epsilon_final_params`` is the paper's final sweep
(``convex_code/experiment_epsilon_final.py:24-315``: 9 nodes, ring, 10 epochs, 5 seeds, random and
label-sorted splits, 9 method x compressor combinations with the tuned step sizes)."""
from __future__ import annotations

import multiprocessing as mp
import os
import pickle

from .data import pickle_it
from .logistic import LogisticDecentralizedSGD
from .parameters import Parameters

_DATA = {}


def _run_one(param):
    m = LogisticDecentralizedSGD(param)
    res = m.fit(_DATA["A"], _DATA["y"])
    print("{} - score: {}".format(param, m.score(_DATA["A"], _DATA["y"])))
    return res


def run_experiment(directory, dataset, params, nproc=None):
    """``dataset`` is a pickle path or an ``(A, y)`` tuple.  Results: ``params.pickle``, ``results.pickle``."""
    os.makedirs(directory, exist_ok=True)
    pickle_it(params, "params", directory)
    if isinstance(dataset, str):
        with open(dataset, "rb") as f:
            A, y = pickle.load(f)
    else:
        A, y = dataset
    _DATA["A"], _DATA["y"] = A, y  # inherited by forked workers
    if nproc and nproc > 1:
        with mp.get_context("fork").Pool(nproc) as pool:
            results = pool.map(_run_one, params)
    else:
        results = [_run_one(p) for p in params]
    pickle_it(results, "results", directory)
    return results


def epsilon_final_params(n=400000, d=2000, n_cores=9, num_epoch=10, seeds=(1, 2, 3, 4, 5), splits=("random", "label-sorted")):
    reg, lr0, tau = 1.0 / n, 0.1, float(d)
    common = dict(num_epoch=num_epoch, lr_type="decay", initial_lr=lr0, tau=tau, regularizer=reg, estimate="final",
                  n_cores=n_cores, topology="ring", distribute_data=True)
    k, levels = 20, 16
    combos = [
        dict(method="plain", quantization="full"),
        dict(method="choco", quantization="top", coordinates_to_keep=k, consensus_lr=0.04),
        dict(method="choco", quantization="random-biased", coordinates_to_keep=k, consensus_lr=0.01),
        dict(method="choco", quantization="qsgd-biased", num_levels=levels, consensus_lr=0.34),
        dict(method="dcd-psgd", quantization="random-unbiased", coordinates_to_keep=k),
        dict(method="dcd-psgd", quantization="qsgd-unbiased", num_levels=levels),
        dict(method="ecd-psgd", quantization="random-unbiased", coordinates_to_keep=k),
        dict(method="ecd-psgd", quantization="qsgd-unbiased", num_levels=levels),
        dict(method="choco", quantization="full", consensus_lr=1.0),
    ]
    out = []
    for split in splits:
        for seed in seeds:
            for c in combos:
                name = "{}-{}-{}-seed{}".format(c["method"], c["quantization"], split, seed)
                out.append(Parameters(name=name, split_data_strategy=split, random_seed=seed,
                                      split_data_random_seed=seed, **common, **c))
    return out


def main(argv=None):
    """``python -m chocosgd_b200.convex.experiment final --dataset data.pickle --out dir [--nproc 10]``."""
    import argparse

    p = argparse.ArgumentParser()
    p.add_argument("sweep", choices=("final",))
    p.add_argument("--dataset", required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--nproc", type=int, default=1)
    p.add_argument("--num_epoch", type=int, default=10)
    p.add_argument("--seeds", default="1,2,3,4,5")
    a = p.parse_args(argv)
    with open(a.dataset, "rb") as f:
        A, y = pickle.load(f)
    params = epsilon_final_params(n=A.shape[0], d=A.shape[1], num_epoch=a.num_epoch,
                                  seeds=tuple(int(s) for s in a.seeds.split(",")))
    run_experiment(a.out, (A, y), params, nproc=a.nproc)


if __name__ == "__main__":
    main()
