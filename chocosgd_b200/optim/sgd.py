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
        # On a GPU the update runs in the fused kernels (capturable in a CUDA graph):
        #   one node                  fused momentum-SGD
        #   complete graph, n > 1     gradient all-reduce + SGD in ONE kernel over the peer mailboxes
        #   other graphs, n > 1       fused SGD + push of x, then wait + weighted neighbour sum (2 kernels)
        self.engine = None
        self.fused_allreduce = False
        want = getattr(conf, "gossip_impl", "auto")
        multi = self.n_nodes > 1 and self._mailbox_ok() and self.n_nodes - 1 <= 16
        self.fused_gossip = False
        if self.device.type == "cuda" and want != "nccl" and multi and not self.is_centralized:
            # D-PSGD: local step + raw push in one kernel, wait + weighted neighbour sum in a second
            self.engine = self.build_algo_engine("dpsgd", "raw")
            self.fused_gossip = True
        elif self.device.type == "cuda" and want != "nccl" and (self.n_nodes == 1 or multi):
            from ..ops.gossip import ALLREDUCE, ChocoEngine, RankBuffers
            from ..parallel.symm import DistributedMailbox, LoopbackMailbox

            self.momentum_buf = torch.zeros_like(self.arena.x)
            z = torch.zeros(32, device=self.device)
            bufs = {self.rank: RankBuffers(self.arena.x, self.arena.g, self.momentum_buf, z, z)}
            self.fused_allreduce = self.n_nodes > 1 and self.is_centralized
            if self.fused_allreduce:
                nbh = {self.rank: {r: 1.0 / self.n_nodes for r in range(self.n_nodes)}}
                mailbox = lambda pw: DistributedMailbox(graph, pw, self.device, group)
            else:
                nbh = {self.rank: {self.rank: 1.0}}
                mailbox = lambda pw: LoopbackMailbox({self.rank: []}, pw, self.device)
            self.engine = ChocoEngine(
                [self.rank], bufs, nbh, self.seg, [g["weight_decay"] for g in self.param_groups],
                ALLREDUCE if self.fused_allreduce else None, mailbox, self.device,
                wait_budget_ms=getattr(conf, "wait_budget_ms", 2000.0),
            )

    @property
    def capturable(self) -> bool:
        return self.engine is not None and (self.n_nodes == 1 or self.fused_allreduce or self.fused_gossip)

    def prepare_step(self):
        self.local_index += 1
        self.engine.set_hyper(self.lr, self.momentum, 0.0, self.nesterov)
        self.n_bits = 32 * self.seg.n_elements
        return self.n_bits

    def launch(self, stream=None):
        if self.fused_gossip:
            self.engine.launch_step(stream)
        elif self.fused_allreduce:
            self.engine.launch_allreduce_sgd(stream)
        else:
            self.engine.launch_sgd_only(True, stream)

    def load_algo_state(self, st):
        if self.engine is not None:
            # the restored momentum buffer counts as initialised; the all-reduce counter stays
            # in step with the (fresh) mailbox flags
            self.engine.per_rank[self.rank]["step"][1] = 1 if self.local_index > 0 else 0

    def step(self, closure=None, **kargs):
        timer, a = self.timer_of(kargs), self.arena
        ep = self.epoch_of(kargs)
        if self.engine is not None:
            with timer("sync.apply_grad", epoch=ep):
                bits = self.prepare_step()
                self.launch()
            if self.n_nodes > 1 and not self.fused_allreduce and not self.fused_gossip:
                with timer("sync.sync", epoch=ep):
                    self.neighbor_exchange().mix_(a.x)
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
