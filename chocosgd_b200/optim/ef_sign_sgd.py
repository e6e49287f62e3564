"""EF-signSGD: error-feedback sign compression, centralized (Karimireddy et al. 2019).

Step (``dl_code/pcode/optim/ef_sign_sgd.py:78-123``): ``p = d' + mem``; own compressed
``delta = ||p_t||_1 / n_t sign(p_t)`` per tensor; ``mem = p - delta``; norms and packed
signs of all ranks are all-gathered, decoded and averaged; ``x -= lr avg``."""
from __future__ import annotations

import torch

from ..compress.reference import SignCodec
from .base import DistributedOptimizer


class EF_SignSGD(DistributedOptimizer):
    timer_labels = (
        "sync.apply_grad",
        "sync.get_data",
        "sync.use_memory",
        "sync.compress",
        "sync.sync",
        "sync.update_memory",
        "sync.decompress",
    )

    def __init__(self, model, conf, graph, group=None):
        super().__init__(model, conf, graph, group)
        self.codec = SignCodec(self.seg)
        self.memory = torch.zeros_like(self.arena.x)
        self.valid = self.arena.valid_mask()
        if self.fused_wanted() and self.n_nodes - 1 <= 16:
            self.engine = self.build_algo_engine("ef_sign_sgd", "sign", complete=True, mem=self.memory)

    def step(self, closure=None, **kargs):
        timer, ep, a = self.timer_of(kargs), self.epoch_of(kargs), self.arena
        if self.engine is not None:
            return self.fused_step(timer, ep, "sync.sync")
        self.local_index += 1
        with timer("sync.apply_grad", epoch=ep):
            d = self.local_direction()
        with timer("sync.use_memory", epoch=ep):
            p = d.add_(self.memory)
        with timer("sync.compress", epoch=ep):
            payload = self.codec.compress(p)
        with timer("sync.update_memory", epoch=ep):
            own = self.codec.decompress(payload)
            self.memory.copy_(p - own)
        with timer("sync.sync", epoch=ep):
            gathered = self.gather_payloads(payload)
        with timer("sync.decompress", epoch=ep):
            avg = torch.zeros_like(a.x)
            for msg in gathered:
                avg.add_(self.codec.decompress(msg))
            avg.div_(len(gathered))
            a.x.add_(avg, alpha=-self.lr)
        self.n_bits = self.codec.n_bits()
        return self.n_bits

    def algo_state(self):
        return {"memory": self.memory}

    def load_algo_state(self, st):
        if "memory" in st:
            self.memory.copy_(st["memory"])
