"""Matrix-form simulator of every distributed algorithm: all ``n`` nodes in one process.

State is held as ``[n, N]`` tensors (row ``i`` = node ``i``), the update rules are the
recurrences the per-rank optimizers must reproduce.  The reference has the same idea in
two places, the convex simulator (``convex_code/logistic.py:181-197``) and the consensus
step-size tuner (``dl_code/pcode/tools/tune_consensus_stepsize.py:53-64``); here it is the
test oracle for the Gloo/NCCL optimizers and for the fused CUDA kernels.

``grad_fn(i, t, x_i) -> flat gradient`` supplies the stochastic gradient of node ``i``.
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np
import torch

from ..compress.reference import Codec
from ..compress.segments import Segments


class LocalSGD:
    """Momentum-SGD direction with per-tensor weight decay, one state row per node.

    d = g + wd x;  buf = d (first call) | mu buf + d;  d' = d + mu buf (Nesterov) | buf
    (``dl_code/pcode/optim/utils.py:13-47``)."""

    def __init__(self, n_nodes: int, segments: Segments, weight_decay, momentum=0.0, nesterov=False):
        self.mu, self.nesterov = float(momentum), bool(nesterov)
        wd = torch.zeros(segments.total, dtype=torch.float32)
        wds = weight_decay if hasattr(weight_decay, "__len__") else [weight_decay] * segments.n_segments
        for s, w in zip(segments.slices(), wds):
            wd[s] = float(w)
        self.wd = wd
        self.buf = [None] * n_nodes

    def direction(self, i: int, x: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
        d = g + self.wd * x
        if self.mu != 0:
            self.buf[i] = d.clone() if self.buf[i] is None else self.mu * self.buf[i] + d
            d = d + self.mu * self.buf[i] if self.nesterov else self.buf[i]
        return d


class Simulator:
    def __init__(
        self,
        algorithm: str,
        w: np.ndarray,
        x0: torch.Tensor,
        segments: Segments,
        codec: Optional[Codec] = None,
        lr: float = 0.1,
        consensus_stepsize: float = 0.5,
        weight_decay=0.0,
        momentum: float = 0.0,
        nesterov: bool = False,
        identical_init: bool = True,
    ):
        self.alg = algorithm
        self.w = torch.as_tensor(np.asarray(w), dtype=torch.float32)
        self.n = self.w.shape[0]
        self.seg = segments
        self.codec = codec
        self.lr, self.gamma = float(lr), float(consensus_stepsize)
        self.x = x0.clone().float().repeat(self.n, 1) if (identical_init and x0.dim() == 1) else x0.clone().float()
        self.local = LocalSGD(self.n, segments, weight_decay, momentum, nesterov)
        self.t = 0
        z = torch.zeros_like(self.x)
        if algorithm == "choco":
            self.x_hat, self.s = z.clone(), z.clone()
        elif algorithm in ("dcd_psgd", "ecd_psgd"):
            # every node keeps a replica of every neighbour, initialised with its own x
            # (dl_code/pcode/optim/dcd_psgd.py:80-89); rows are identical at start.
            self.rep = self.x.clone()  # rep[j] = the (shared) public copy of node j
        elif algorithm == "deep_squeeze":
            self.mem = z.clone()
        elif algorithm in ("dgc", "ef_sign_sgd"):
            self.mem = z.clone()

    # -- helpers ---------------------------------------------------------------------------
    def _q(self, v: torch.Tensor, node: int) -> torch.Tensor:
        return self.codec.roundtrip(v, self.t, node) if self.codec is not None else v.clone()

    def _mix(self, m: torch.Tensor) -> torch.Tensor:
        return self.w @ m

    def step(self, grad_fn: Callable[[int, int, torch.Tensor], torch.Tensor]):
        n, lr = self.n, self.lr
        dirs = torch.stack([self.local.direction(i, self.x[i], grad_fn(i, self.t, self.x[i])) for i in range(n)])
        alg = self.alg
        if alg == "centralized_sgd":
            # gradients are averaged *before* the local momentum step (sgd.py:68-92)
            raise RuntimeError("use step_centralized for centralized_sgd")
        if alg == "dpsgd":
            self.x = self._mix(self.x - lr * dirs)
        elif alg == "choco":
            xh = self.x - lr * dirs
            xn = xh + self.gamma * (self.s - self.x_hat)
            q = torch.stack([self._q(xn[i] - self.x_hat[i], i) for i in range(n)])
            self.x_hat = self.x_hat + q
            self.s = self.s + self._mix(q)
            self.x = xn
        elif alg == "dcd_psgd":
            half = self._mix(self.rep) - lr * dirs
            q = torch.stack([self._q(half[i] - self.x[i], i) for i in range(n)])
            self.rep = self.rep + q
            self.x = self.rep.clone()
        elif alg == "ecd_psgd":
            t = float(self.t + 1)  # conf.local_index starts at 1 on the first step
            x_new = self._mix(self.rep) - lr * dirs
            z = (1 - 0.5 * t) * self.x + 0.5 * t * x_new
            self._ecd_update(z, t)
            self.x = x_new
        elif alg == "deep_squeeze":
            xh = self.x - lr * dirs
            self.mem = self.mem + xh
            c = torch.stack([self._q(self.mem[i], i) for i in range(n)])
            self.mem = self.mem - c
            self.x = xh + self.gamma * ((self.w - torch.eye(n)) @ c)
        elif alg == "ef_sign_sgd":
            p = dirs * 1.0 + self.mem
            delta = torch.stack([self._q(p[i], i) for i in range(n)])
            self.mem = p - delta
            self.x = self.x - lr * delta.mean(dim=0, keepdim=True)
        elif alg == "dgc":
            v = dirs + self.mem
            sel = torch.stack([self._q(v[i], i) for i in range(n)])
            self.mem = v - sel
            self.x = self.x - lr * sel.mean(dim=0, keepdim=True)
        else:
            raise NotImplementedError(alg)
        self.t += 1

    def _ecd_update(self, z: torch.Tensor, t: float):
        codec = self.codec
        for j in range(self.n):
            if codec is not None and codec.is_sparse:
                pos, val = codec.sparse(codec.compress(z[j], self.t, j), self.t, j)
                self.rep[j, pos] = (1 - 2 / t) * self.rep[j, pos] + (2 / t) * val
            else:
                q = self._q(z[j], j)
                self.rep[j] = (1 - 2 / t) * self.rep[j] + (2 / t) * q

    def step_centralized(self, grad_fn):
        """All-reduce-average SGD: grads averaged, then one momentum step per node."""
        g = torch.stack([grad_fn(i, self.t, self.x[i]) for i in range(self.n)]).mean(dim=0)
        for i in range(self.n):
            self.x[i] = self.x[i] - self.lr * self.local.direction(i, self.x[i], g)
        self.t += 1

    # -- diagnostics -------------------------------------------------------------------------
    def consensus_error(self) -> float:
        xbar = self.x.mean(dim=0, keepdim=True)
        return float(((self.x - xbar) ** 2).sum())


def choco_gossip_error(w, codec_fn, gamma, n_params=1000, n_iters=1000, seed=0):
    """Error of pure CHOCO-Gossip (no gradients) after ``n_iters`` rounds, starting from
    X ~ N(0, 1):  X += gamma X_hat (W - I);  X_hat += Q(X - X_hat);  error =
    sum ||x_i - xbar||^2 + sum ||x_i - x_hat_i||^2
    (``dl_code/pcode/tools/tune_consensus_stepsize.py:53-64``)."""
    g = torch.Generator().manual_seed(seed)
    wt = torch.as_tensor(np.asarray(w), dtype=torch.float32)
    n = wt.shape[0]
    x = torch.randn(n, n_params, generator=g)
    xh = torch.zeros_like(x)
    eye = torch.eye(n)
    for t in range(n_iters):
        x = x + gamma * ((wt - eye) @ xh)
        q = torch.stack([codec_fn(x[i] - xh[i], t) for i in range(n)])
        xh = xh + q
        if not torch.isfinite(x).all():
            return float("inf")
    xbar = x.mean(dim=0, keepdim=True)
    return float(((x - xbar) ** 2).sum() + ((x - xh) ** 2).sum())
