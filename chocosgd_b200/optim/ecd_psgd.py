"""ECD-PSGD: extrapolation-compression decentralized SGD (Tang et al. 2018).

With ``t`` the 1-based step index (``dl_code/pcode/optim/ecd_psgd.py:99-157``)::

    x_new = sum_j w_ij x_hat_j - lr d'           (becomes the model)
    z     = (1 - t/2) x_old + (t/2) x_new
    q_i   = Q(z)   (the tensor itself, not a difference), exchanged with the neighbours
    x_hat_j <- (1 - 2/t) x_hat_j + (2/t) q_j     (sparse codecs: only at received indices)
"""
from __future__ import annotations

import torch

from .base import DistributedOptimizer


class ECD_PSGD(DistributedOptimizer):
    timer_labels = (
        "grad.apply_grad",
        "grad.get_params",
        "grad.get_extrapolated_model",
        "grad.unflatten_to_update",
        "grad.compress",
        "grad.sync",
    )

    def __init__(self, model, conf, graph, group=None):
        super().__init__(model, conf, graph, group)
        self.codec = self.make_codec()
        self.neighbor_hat_params = {r: self.arena.x.clone() for r in self.neighbors_info}
        if self.fused_wanted():
            self.engine = self.build_algo_engine("ecd_psgd", conf.comm_op, hats=self.neighbor_hat_params)

    def step(self, closure=None, **kargs):
        timer, ep, a = self.timer_of(kargs), self.epoch_of(kargs), self.arena
        if self.engine is not None:
            return self.fused_step(timer, ep, "grad.sync")
        step = self.local_index
        self.local_index += 1
        t = float(self.local_index)
        with timer("grad.apply_grad", epoch=ep):
            d = self.local_direction()
        with timer("grad.get_extrapolated_model", epoch=ep):
            x_new = sum(hat * self.neighbors_info[r] for r, hat in self.neighbor_hat_params.items())
            x_new = x_new.add(d, alpha=-self.lr)
            z = (1 - 0.5 * t) * a.x + (0.5 * t) * x_new
        with timer("grad.unflatten_to_update", epoch=ep):
            a.x.copy_(x_new)
        with timer("grad.compress", epoch=ep):
            payload = self.codec.compress(z, step, self.rank)
        with timer("grad.sync", epoch=ep):
            received = self.neighbor_exchange()._agg(payload, op="get_raw_sync_data")
        with timer("grad.unflatten_to_update", epoch=ep):
            for rank in self.neighbors_info:
                hat = self.neighbor_hat_params[rank]
                if self.codec.is_sparse:
                    pos, val = self.codec.sparse(received[rank], step, rank)
                    hat[pos] = hat[pos] * (1 - 2 / t) + (2 / t) * val
                else:
                    hat.mul_(1 - 2 / t).add_(self.codec.decompress(received[rank], step, rank), alpha=2 / t)
        self.n_bits = self.codec.n_bits()
        return self.n_bits

    def algo_state(self):
        return {f"hat_{r}": t for r, t in self.neighbor_hat_params.items()}

    def load_algo_state(self, st):
        for r in self.neighbor_hat_params:
            if f"hat_{r}" in st:
                self.neighbor_hat_params[r].copy_(st[f"hat_{r}"])
