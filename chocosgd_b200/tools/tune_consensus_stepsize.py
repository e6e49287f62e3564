"""Grid search of the CHOCO consensus step size gamma by simulating CHOCO-Gossip.

Start from X ~ N(0,1)^{n x d}, iterate ``X += gamma (W - I) X_hat ; X_hat += Q(X - X_hat)``
and score ``sum ||x_i - xbar||^2 + sum ||x_i - x_hat_i||^2`` after ``n_iters`` rounds; the
best gamma of ``logspace(-3, 0, n_grid)`` wins.  Same procedure as
``dl_code/pcode/tools/tune_consensus_stepsize.py:53-97`` (which cannot be imported as
shipped: it imports a method as a module function and passes wrong keyword names).

    python -m chocosgd_b200.tools.tune_consensus_stepsize --graph_topology ring --n_nodes 8 \
        --comm_op compress_top_k --compress_ratio 0.99
"""
from __future__ import annotations

import argparse
from functools import partial
from multiprocessing import Pool

import numpy as np
import torch

from ..compress.reference import make_codec
from ..compress.segments import Segments
from ..parallel.topology import mixing_matrix
from ..sim.matrix_form import choco_gossip_error


def evaluate_gamma(gamma, topology, n_nodes, comm_op, compress_ratio, quantize_level, is_biased, n_params, n_iters,
                   seed):
    torch.set_num_threads(1)
    seg = Segments.from_sizes([n_params])
    codec = make_codec(seg, comm_op, compress_ratio, quantize_level, None, is_biased, seed)
    pad = seg.total - n_params

    def q(v, t):
        full = torch.cat([v, v.new_zeros(pad)]) if pad else v
        return codec.roundtrip(full, t)[:n_params]

    return choco_gossip_error(mixing_matrix(topology, n_nodes), q, float(gamma), n_params, n_iters, seed)


def search_gamma(topology="ring", n_nodes=8, comm_op="compress_top_k", compress_ratio=0.99, quantize_level=4,
                 is_biased=False, n_params=1000, n_iters=1000, n_grid=20, seed=0, n_proc=4):
    gammas = np.logspace(-3, 0, n_grid)
    fn = partial(evaluate_gamma, topology=topology, n_nodes=n_nodes, comm_op=comm_op, compress_ratio=compress_ratio,
                 quantize_level=quantize_level, is_biased=is_biased, n_params=n_params, n_iters=n_iters, seed=seed)
    if n_proc > 1:
        with Pool(n_proc) as pool:
            errors = pool.map(fn, gammas)
    else:
        errors = [fn(g) for g in gammas]
    errors = [e if np.isfinite(e) else float("inf") for e in errors]
    best = int(np.argmin(errors))
    return float(gammas[best]), list(zip(gammas.tolist(), errors))


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--graph_topology", default="ring")
    p.add_argument("--n_nodes", type=int, default=8)
    p.add_argument("--comm_op", default="compress_top_k")
    p.add_argument("--compress_ratio", type=float, default=0.99)
    p.add_argument("--quantize_level", type=int, default=4)
    p.add_argument("--is_biased", action="store_true")
    p.add_argument("--n_params", type=int, default=1000)
    p.add_argument("--n_iters", type=int, default=1000)
    p.add_argument("--n_grid", type=int, default=20)
    p.add_argument("--n_proc", type=int, default=4)
    a = p.parse_args(argv)
    best, table = search_gamma(a.graph_topology, a.n_nodes, a.comm_op, a.compress_ratio, a.quantize_level,
                               a.is_biased, a.n_params, a.n_iters, a.n_grid, 0, a.n_proc)
    for g, e in table:
        print(f"gamma {g:.5f}  error {e:.4e}")
    print(f"best consensus_stepsize: {best:.5f}")
    return best


if __name__ == "__main__":
    main()
