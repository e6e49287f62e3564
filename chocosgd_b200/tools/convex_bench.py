"""Convex plumbing run on the CPU (``--device cuda``: the same recurrences with one kernel per iteration): L2-regularised logistic regression (lambda = 1/N) with CHOCO-SGD
(top-k, k = 1 % of d) against exact decentralized SGD, 9 simulated nodes on a ring, synthetic data
(``convex_code/logistic.py``, ``convex_code/experiment_epsilon_final.py:24-60``).

    python -m chocosgd_b200.tools.convex_bench --samples 40000 --features 2000 --epochs 2
"""
from __future__ import annotations

import argparse
import json
import time


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--samples", type=int, default=40000)
    p.add_argument("--features", type=int, default=2000)
    p.add_argument("--nodes", type=int, default=9)
    p.add_argument("--epochs", type=int, default=2)
    p.add_argument("--device", default="cpu", help="cpu (numpy) or cuda (one kernel per simulator iteration)")
    a = p.parse_args(argv)
    from ..convex import LogisticDecentralizedSGD, Parameters
    from ..convex.data import synthetic_logistic

    A, y = synthetic_logistic(a.samples, a.features, seed=0, noise=0.1)
    n, d = A.shape
    k = max(1, d // 100)
    if a.device != "cpu":
        # context creation, library load and the first transfers are not part of an iteration's cost
        warm = Parameters(num_epoch=1, lr_type="decay", initial_lr=0.1, tau=float(d), regularizer=1.0 / n, estimate="final",
                          n_cores=a.nodes, topology="ring", distribute_data=True, split_data_strategy="random",
                          method="choco", quantization="top", coordinates_to_keep=k, consensus_lr=0.04, random_seed=1,
                          split_data_random_seed=1)
        LogisticDecentralizedSGD(warm, device=a.device).fit(A[: 50 * a.nodes], y[: 50 * a.nodes])
    for method, quant, extra in (("choco", "top", dict(coordinates_to_keep=k, consensus_lr=0.04)), ("plain", "full", {})):
        prm = Parameters(num_epoch=a.epochs, lr_type="decay", initial_lr=0.1, tau=float(d), regularizer=1.0 / n,
                         estimate="final", n_cores=a.nodes, topology="ring", distribute_data=True,
                         split_data_strategy="random", method=method, quantization=quant, random_seed=1,
                         split_data_random_seed=1, **extra)
        m = LogisticDecentralizedSGD(prm, device=a.device)
        t0 = time.time()
        m.fit(A, y)
        dt = time.time() - t0
        iters = a.epochs * n // a.nodes
        print(json.dumps({"bench": "convex", "device": a.device, "samples": n, "features": d, "nodes": a.nodes, "topology": "ring",
                          "epochs": a.epochs, "method": method, "quantization": quant, "k": k if quant == "top" else None,
                          "seconds": round(dt, 2), "iterations": iters,
                          "us_per_iteration_all_nodes": round(1e6 * dt / iters, 1),
                          "final_loss": float(m.loss(A, y)), "train_accuracy": float(m.score(A, y))}), flush=True)


if __name__ == "__main__":
    main()
