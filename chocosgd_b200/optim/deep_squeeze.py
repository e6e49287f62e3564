"""DeepSqueeze: error-compensated compressed gossip (Tang et al. 2019).

Error memory ``e`` starts at zero (``dl_code/pcode/optim/deep_squeeze.py:82-127``)::

    x <- x - lr d' ;  e <- e + x ;  c_i = Q(e) ;  e <- e - c_i
    exchange c ;  x <- x + gamma sum_j (w_ij - [j == i]) c_j
"""
from __future__ import annotations

import torch

from .base import DistributedOptimizer


class DeepSqueeze(DistributedOptimizer):
    timer_labels = (
        "grad.apply_grad",
        "grad.get_params",
        "grad.error_compensate",
        "grad.compress",
        "grad.update_memory",
        "grad.sync",
        "grad.decompress",
    )

    def __init__(self, model, conf, graph, group=None):
        super().__init__(model, conf, graph, group)
        self.codec = self.make_codec()
        self.consensus_stepsize = float(conf.consensus_stepsize)
        self.memory = torch.zeros_like(self.arena.x)
        self.gamma_for_engine = self.consensus_stepsize
        if self.fused_wanted():
            self.engine = self.build_algo_engine("deep_squeeze", conf.comm_op, mem=self.memory)

    def step(self, closure=None, **kargs):
        timer, ep, a = self.timer_of(kargs), self.epoch_of(kargs), self.arena
        if self.engine is not None:
            return self.fused_step(timer, ep, "grad.sync")
        step = self.local_index
        self.local_index += 1
        with timer("grad.apply_grad", epoch=ep):
            a.x.add_(self.local_direction(), alpha=-self.lr)
        with timer("grad.error_compensate", epoch=ep):
            self.memory.add_(a.x)
        with timer("grad.compress", epoch=ep):
            payload = self.codec.compress(self.memory, step, self.rank)
        with timer("grad.update_memory", epoch=ep):
            self.memory.sub_(self.codec.decompress(payload, step, self.rank))
        with timer("grad.sync", epoch=ep):
            received = self.neighbor_exchange()._agg(payload, op="get_raw_sync_data")
        with timer("grad.decompress", epoch=ep):
            for rank, w in self.neighbors_info.items():
                coeff = self.consensus_stepsize * (w - (1.0 if rank == self.rank else 0.0))
                if self.codec.is_sparse:
                    pos, val = self.codec.sparse(received[rank], step, rank)
                    a.x.index_add_(0, pos, val, alpha=coeff)
                else:
                    a.x.add_(self.codec.decompress(received[rank], step, rank), alpha=coeff)
        self.n_bits = self.codec.n_bits()
        return self.n_bits

    def algo_state(self):
        return {"memory": self.memory}

    def load_algo_state(self, st):
        if "memory" in st:
            self.memory.copy_(st["memory"])
