"""Deep Gradient Compression (centralized, all-gather of sparse gradients).

Step (``dl_code/pcode/optim/dgc.py:118-324``): momentum direction ``d'`` with optional
per-tensor norm clipping scaled by 1/sqrt(n) applied *before* the momentum update
(``:254-265,300-302``); ``v = d' + mem``; per-tensor top-/random-k at the (warm-up) ratio;
``mem = v`` outside the selection, optional momentum-factor masking; all ranks' selections
are all-gathered, scatter-added, divided by n and applied with the learning rate.  With a
quantizer instead of a sparsifier the quantized gradients are all-reduced and no memory is
kept.

The reference computes the residual with a bitwise NOT of a ``uint8`` mask
(``dl_code/pcode/utils/sparsification.py:33-38``), which on torch >= 1.2 yields factors
254/255 instead of 0/1 and makes the memory explode; the intended ``mem = v (1 - mask)``
is implemented here.  First momentum call: ``buf = d`` (``:313-315``)."""
from __future__ import annotations

import math

import torch

from ..compress.reference import make_codec
from .base import DistributedOptimizer


class DGC(DistributedOptimizer):
    timer_labels = (
        "grad.apply_grad",
        "grad.recover_hat_params",
        "grad.compress",
        "grad.sync",
        "grad.recover_info",
        "grad.update_model",
    )

    def __init__(self, model, conf, graph, group=None):
        super().__init__(model, conf, graph, group)
        self.comm_op = conf.comm_op
        self.is_compress_op = "compress" in conf.comm_op
        self.compress_ratio = conf.compress_ratio
        self.compress_warmup_epochs = conf.compress_warmup_epochs
        self.mask_momentum = conf.mask_momentum
        self.clip_grad = conf.clip_grad
        self.clip_grad_val = conf.clip_grad_val
        self.memory = torch.zeros_like(self.arena.x)
        if self.is_compress_op:
            vals = [float(v) for v in conf.compress_warmup_values.split(",")]
            self.compress_warmup_values = [v for v in vals if v <= self.compress_ratio]
            n = len(self.compress_warmup_values)
            self.detailed_compress_warmup_epochs = [
                1.0 * i / n * self.compress_warmup_epochs for i in range(1, n + 1)
            ]
        self._codecs = {}
        # Fused kernels: whenever the selection size is fixed for the whole run (no sparsity
        # warm-up) and no per-tensor clipping is asked for; otherwise the PyTorch statement below.
        static_ratio = not self.is_compress_op or self.compress_warmup_epochs <= 0
        if (self.fused_wanted() and static_ratio and not self.clip_grad and self.n_nodes - 1 <= 16
                and conf.comm_op in ("compress_top_k", "compress_random_k", "quantize_qsgd")
                and not (conf.comm_op == "quantize_qsgd" and (conf.quantize_level or 0) >= 32)):
            self.codec = self._codec(self._get_compress_ratio(0.0))
            self.engine = self.build_algo_engine(
                "dgc", conf.comm_op, complete=True, mem=self.memory if self.is_compress_op else None,
                mask_momentum=bool(self.mask_momentum), use_memory=self.is_compress_op)

    def _get_compress_ratio(self, epoch_):
        if not self.is_compress_op:
            return None
        if epoch_ < self.compress_warmup_epochs:
            for ind, val in enumerate(self.detailed_compress_warmup_epochs):
                if epoch_ < val:
                    return self.compress_warmup_values[ind]
        return self.compress_ratio

    def _codec(self, ratio):
        if ratio not in self._codecs:
            self._codecs[ratio] = self.make_codec(compress_ratio=ratio)
        return self._codecs[ratio]

    def _direction(self):
        a = self.arena
        d = torch.addcmul(a.g, self.wd_vec, a.x)
        if self.clip_grad and self.clip_grad_val is not None:
            thr = self.clip_grad_val / math.sqrt(self.n_nodes)
            for sl in self.seg.slices():
                nrm = d[sl].norm(p=2)
                if nrm >= thr:
                    d[sl].mul_(thr / nrm)
        mu = self.momentum
        if mu != 0:
            if self.momentum_buf is None:
                self.momentum_buf = d.clone()
            else:
                self.momentum_buf.mul_(mu).add_(d)
            d = d.add(self.momentum_buf, alpha=mu) if self.nesterov else self.momentum_buf.clone()
        a.g.zero_()
        return d

    def step(self, closure=None, **kargs):
        timer, ep, a = self.timer_of(kargs), self.epoch_of(kargs), self.arena
        if self.engine is not None:
            return self.fused_step(timer, ep, "grad.sync")
        step = self.local_index
        self.local_index += 1
        with timer("grad.apply_grad", epoch=ep):
            d = self._direction()
        codec = self._codec(self._get_compress_ratio(ep))
        with timer("grad.compress", epoch=ep):
            if self.is_compress_op:
                v = d + self.memory
                payload = codec.compress(v, step, self.rank)
                pos, _ = codec.sparse(payload, step, self.rank)
                self.memory.copy_(v)
                self.memory[pos] = 0
                if self.mask_momentum and self.momentum_buf is not None:
                    self.momentum_buf[pos] = 0
            else:
                payload = codec.compress(d, step, self.rank)
        with timer("grad.sync", epoch=ep):
            if self.is_compress_op:
                gathered = self.gather_payloads(payload)
            else:
                dense = codec.decompress(payload, step, self.rank)
                gathered = self.world_aggregator._agg(dense, op="sum", communication_scheme="all_reduce")
        with timer("grad.recover_info", epoch=ep):
            if self.is_compress_op:
                update = torch.zeros_like(a.x)
                for r, msg in enumerate(gathered):
                    src = r if len(gathered) > 1 else self.rank
                    p, val = codec.sparse(msg, step, src)
                    update.index_add_(0, p, val)
                update.div_(self.n_nodes)
            else:
                update = gathered / self.n_nodes
        with timer("grad.update_model", epoch=ep):
            a.x.add_(update, alpha=-self.lr)
        self.n_bits = codec.n_bits()
        return self.n_bits

    def algo_state(self):
        return {"memory": self.memory}

    def load_algo_state(self, st):
        if "memory" in st:
            self.memory.copy_(st["memory"])
