"""DCD-PSGD: difference-compression decentralized SGD (Tang et al. 2018).

Every rank keeps a replica ``x_hat_j`` of each neighbour **and of itself**, all initialised
with its own parameters (``dl_code/pcode/optim/dcd_psgd.py:80-89``).  Step (``:96-144``)::

    half = sum_j w_ij x_hat_j - lr d'
    q_i  = Q(half - x_i)              exchanged (blocking) with the neighbours
    x_hat_j += q_j  for all j in N(i) (self included);  x_i <- x_hat_i
"""
from __future__ import annotations

import torch

from .base import DistributedOptimizer


class DCD_PSGD(DistributedOptimizer):
    timer_labels = (
        "grad.apply_grad",
        "grad.get_grads",
        "grad.apply_local_gradient",
        "grad.compress",
        "grad.sync",
        "grad.unflatten_to_update",
    )

    def __init__(self, model, conf, graph, group=None):
        super().__init__(model, conf, graph, group)
        self.codec = self.make_codec()
        self.neighbor_hat_params = {r: self.arena.x.clone() for r in self.neighbors_info}
        if self.fused_wanted():
            self.engine = self.build_algo_engine("dcd_psgd", conf.comm_op, hats=self.neighbor_hat_params)

    def _apply(self, received, step):
        for rank in self.neighbors_info:
            hat = self.neighbor_hat_params[rank]
            if self.codec.is_sparse:
                pos, val = self.codec.sparse(received[rank], step, rank)
                hat.index_add_(0, pos, val)
            else:
                hat.add_(self.codec.decompress(received[rank], step, rank))

    def step(self, closure=None, **kargs):
        timer, ep, a = self.timer_of(kargs), self.epoch_of(kargs), self.arena
        if self.engine is not None:
            return self.fused_step(timer, ep, "grad.sync")
        step = self.local_index
        self.local_index += 1
        with timer("grad.apply_grad", epoch=ep):
            d = self.local_direction()
        with timer("grad.apply_local_gradient", epoch=ep):
            half = sum(hat * self.neighbors_info[r] for r, hat in self.neighbor_hat_params.items())
            half = half.add(d, alpha=-self.lr)
        with timer("grad.compress", epoch=ep):
            payload = self.codec.compress(half - a.x, step, self.rank)
        with timer("grad.sync", epoch=ep):
            received = self.neighbor_exchange()._agg(payload, op="get_raw_sync_data")
        with timer("grad.unflatten_to_update", epoch=ep):
            self._apply(received, step)
            a.x.copy_(self.neighbor_hat_params[self.rank])
        self.n_bits = self.codec.n_bits()
        return self.n_bits

    def algo_state(self):
        return {f"hat_{r}": t for r, t in self.neighbor_hat_params.items()}

    def load_algo_state(self, st):
        for r in self.neighbor_hat_params:
            if f"hat_{r}" in st:
                self.neighbor_hat_params[r].copy_(st[f"hat_{r}"])
