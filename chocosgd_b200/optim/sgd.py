"""Centralized (all-reduce) SGD and decentralized D-PSGD.

``complete`` topology: gradients are averaged over all ranks, then one local
momentum-SGD step (``dl_code/pcode/optim/sgd.py:68-92``).  Any other topology: local step
first, then full-precision gossip averaging ``x_i <- sum_j w_ij x_j`` with the graph
neighbours (``:93-121``)."""
from __future__ import annotations

import torch

from .base import DistributedOptimizer


class SGD(DistributedOptimizer):
    timer_labels = ("sync.get_data", "sync.sync", "sync.unflatten_grad", "sync.apply_grad", "sync.update_model")

    def __init__(self, model, conf, graph, group=None, is_centralized=None):
        super().__init__(model, conf, graph, group)
        self.is_centralized = (conf.graph_topology == "complete") if is_centralized is None else is_centralized
        # single node on a GPU: the whole update is one fused kernel (capturable in a CUDA graph)
        self.engine = None
        want = getattr(conf, "gossip_impl", "auto")
        if self.n_nodes == 1 and self.device.type == "cuda" and want != "nccl":
            from ..ops.gossip import ChocoEngine, RankBuffers
            from ..parallel.symm import LoopbackMailbox

            self.momentum_buf = torch.zeros_like(self.arena.x)
            z = torch.zeros(32, device=self.device)
            bufs = {self.rank: RankBuffers(self.arena.x, self.arena.g, self.momentum_buf, z, z)}
            self.engine = ChocoEngine(
                [self.rank], bufs, {self.rank: {self.rank: 1.0}}, self.seg,
                [g["weight_decay"] for g in self.param_groups], None,
                lambda pw: LoopbackMailbox({self.rank: []}, pw, self.device), self.device,
            )

    @property
    def capturable(self) -> bool:
        return self.engine is not None

    def prepare_step(self):
        self.local_index += 1
        self.engine.set_hyper(self.lr, self.momentum, 0.0, self.nesterov)
        self.n_bits = 32 * self.seg.n_elements
        return self.n_bits

    def launch(self, stream=None):
        self.engine.launch_sgd_only(True, stream)

    def step(self, closure=None, **kargs):
        timer, a = self.timer_of(kargs), self.arena
        ep = self.epoch_of(kargs)
        if self.engine is not None:
            with timer("sync.apply_grad", epoch=ep):
                bits = self.prepare_step()
                self.launch()
            return bits
        self.local_index += 1
        if self.is_centralized:
            with timer("sync.sync", epoch=ep):
                if self.n_nodes > 1:
                    a.g.copy_(self.world_aggregator._agg(a.g, op="avg"))
            with timer("sync.apply_grad", epoch=ep):
                a.x.add_(self.local_direction(), alpha=-self.lr)
        else:
            with timer("sync.apply_grad", epoch=ep):
                a.x.add_(self.local_direction(), alpha=-self.lr)
            with timer("sync.sync", epoch=ep):
                if self.n_nodes > 1:
                    ex = self.neighbor_exchange()
                    if hasattr(ex, "mix_"):
                        ex.mix_(a.x)  # push + fused wait / weighted sum, no library call
                    else:
                        mixed = ex._agg(a.x, op="weighted")
                        with timer("sync.update_model", epoch=ep):
                            a.x.copy_(mixed)
        self.n_bits = 32 * self.seg.n_elements
        return self.n_bits
