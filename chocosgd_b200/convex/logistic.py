"""Matrix-form simulation of decentralized SGD on L2-regularised logistic regression.

State is ``x in R^{d x n}`` (column m = node m).  Per iteration every node samples one of its
rows and takes a gradient step ``Delta_m = lr_t (y a sigma(-y a.x_m) - lambda x_m)``, then::

    plain      x <- (x + Delta) W
    choco      x <- x + Delta + gamma x_hat (W - I) ;  x_hat += Q(x - x_hat)
    dcd-psgd   x += Q(x W + Delta - x)
    ecd-psgd   x_new = x_hat W + Delta ;  z = (1 - (t+1)/2) x + (t+1)/2 x_new ;
               x <- x_new ;  x_hat <- (1 - 2/(t+1)) x_hat + 2/(t+1) Q(z)

(``convex_code/logistic.py:97-209``; there x_hat starts equal to x, unlike the deep-learning
code where it starts at zero).  The loss of the node-averaged iterate is logged ten times per
epoch.  All random draws go through one ``numpy.random.RandomState`` in the order
sample(node 0..n-1), then the compressor's draws column by column, so a run is a pure
function of ``random_seed``.

``device="cuda"`` runs the same recurrences with the state on the GPU (row sampling and
compressor randomness stay on the host RNG, so both devices follow the same trajectory up to
floating-point rounding)."""
from __future__ import annotations

import time

import numpy as np

from .parameters import Parameters

INIT_WEIGHT_STD = 0.01
LOSS_PER_EPOCH = 10


def sigmoid(z):
    return 0.5 * (1.0 + np.tanh(0.5 * z))


def qsgd_quantize(x, s, is_biased, rs=np.random):
    """QSGD with ``s`` levels on one vector (``convex_code/logistic.py:13-23``)."""
    norm = np.sqrt(np.sum(np.square(x)))
    if norm == 0:
        rs.rand(*x.shape)
        return np.zeros_like(x)
    level = s * np.abs(x) / norm
    low = np.floor(level)
    new_level = low + (rs.rand(*x.shape) < (level - low))
    scale = 1.0
    if is_biased:
        n = len(x)
        scale = 1.0 / (min(n / s ** 2, np.sqrt(n) / s) + 1.0)
    return scale * np.sign(x) * norm * new_level / s


def mixing_matrix_convex(topology, n):
    if topology == "ring":
        w = np.zeros((n, n))
        v = 1.0 / 3 if n >= 3 else 1.0 / 2
        for i in range(n):
            w[i, i] = v
            if n > 1:
                w[i, (i + 1) % n] = v
                w[i, (i - 1) % n] = v
        return w
    if topology == "centralized":
        return np.ones((n, n)) / n
    if topology == "disconnected":
        return np.eye(n)
    if topology == "torus":
        side = int(np.sqrt(n))
        if side * side != n:
            raise ValueError("torus needs a square number of nodes")
        from ..parallel.topology import torus_matrix

        return torus_matrix(n)
    raise ValueError(topology)


class LogisticDecentralizedSGD:
    def __init__(self, params: Parameters, device: str = "cpu", verbose: bool = False):
        self.params = params
        self.x = None
        self.x_estimate = None
        self.x_hat = None
        self.W = mixing_matrix_convex(params.topology, params.n_cores)
        self.device = device
        self.verbose = verbose
        self.transmitted_bits = 0.0

    # ---- schedules / estimates ------------------------------------------------------------------
    def lr(self, epoch, iteration, num_samples, d):
        p = self.params
        t = epoch * num_samples + iteration
        if p.lr_type == "constant":
            return p.initial_lr
        if p.lr_type == "epoch-decay":
            return p.initial_lr * (p.epoch_decay_lr ** epoch)
        if p.lr_type == "decay":
            return p.initial_lr / (p.regularizer * (t + p.tau))
        return p.initial_lr / (1 + p.initial_lr * p.regularizer * t)  # bottou

    def update_estimate(self, t):
        t, p = int(t), self.params
        if p.estimate == "final":
            self.x_estimate = self.x
            return
        if p.estimate == "mean":
            rho = 1 / (t + 1)
        elif p.estimate == "t+tau":
            rho = 2 * (t + p.tau) / ((1 + t) * (t + 2 * p.tau))
        else:
            rho = 6 * ((t + p.tau) ** 2) / ((1 + t) * (6 * (p.tau ** 2) + t + 6 * p.tau * t + 2 * (t ** 2)))
        self.x_estimate = self.x_estimate * (1 - rho) + self.x * rho

    def _mean_iterate(self):
        x = self.x_estimate if self.x_estimate is not None else self.x
        return np.asarray(x).mean(axis=1)

    def loss(self, A, y):
        x = self._mean_iterate()
        z = -y * (A @ x)
        out = np.sum(np.logaddexp(0.0, z)) / A.shape[0]
        if self.params.regularizer:
            out += self.params.regularizer * np.square(x).sum() / 2
        return float(out)

    def predict(self, A):
        return 1 * ((A @ self._mean_iterate()) >= 0.0)

    def predict_proba(self, A):
        return sigmoid(A @ self._mean_iterate())

    def score(self, A, y):
        pred = 2 * ((A @ self._mean_iterate()) >= 0.0) - 1
        return float(np.mean(pred == y))

    # ---- compression ---------------------------------------------------------------------------------
    def bits_per_node_iteration(self, d):
        """Bit model of the reference's plots (``convex_code/plots-epsilon.ipynb:89-95``)."""
        p, q = self.params, self.params.quantization
        if q == "full":
            return 64 * 2 * d
        if q.startswith("random"):
            return 64 * 2 * p.coordinates_to_keep
        if q == "top":
            return (64 + int(np.ceil(np.log2(d)))) * 2 * p.coordinates_to_keep
        return (int(np.ceil(np.log2(p.num_levels))) + 1) * 2 * d

    def quantize(self, x, rs):
        """Column-wise compressor on ``x`` of shape (d, n)."""
        p, q = self.params, self.params.quantization
        if q == "full":
            return x
        out = np.zeros_like(x)
        if q in ("qsgd-biased", "qsgd-unbiased"):
            for i in range(x.shape[1]):
                out[:, i] = qsgd_quantize(x[:, i], p.num_levels, q == "qsgd-biased", rs)
            return out
        k = p.coordinates_to_keep
        if q == "top":
            for i in range(x.shape[1]):
                idx = np.argsort(np.abs(x[:, i]))[::-1][:k]
                out[idx, i] = x[idx, i]
            return out
        for i in range(x.shape[1]):
            idx = rs.choice(np.arange(x.shape[0]), k, replace=False)
            out[idx, i] = x[idx, i]
        return x.shape[0] / k * out if q == "random-unbiased" else out

    # ---- data split ---------------------------------------------------------------------------------
    def split_indices(self, y, num_samples):
        p = self.params
        if not p.distribute_data:
            return num_samples, [np.arange(num_samples) for _ in range(p.n_cores)]
        rs = np.random.RandomState(p.split_data_random_seed)
        per = num_samples // p.n_cores
        if p.split_data_strategy == "random":
            order = np.arange(num_samples)
            rs.shuffle(order)
        elif p.split_data_strategy == "naive":
            order = np.arange(num_samples)
        else:
            order = np.argsort(y)
        idx = [order[per * m: per * (m + 1)] for m in range(p.n_cores - 1)]
        idx.append(order[per * (p.n_cores - 1):])
        return per, idx

    # ---- training -------------------------------------------------------------------------------------
    def fit(self, A, y_init):
        """-> (loss after every epoch [num_epoch + 1], loss trace with 10 points per epoch)."""
        if self.device != "cpu":
            return self._fit_torch(A, y_init)
        p = self.params
        y = np.copy(y_init)
        num_samples, d = A.shape
        n = p.n_cores
        rs = np.random.RandomState(p.random_seed)
        if self.x is None:
            x0 = np.random.RandomState(p.random_seed).normal(0, INIT_WEIGHT_STD, size=(d,)) if p.random_seed is not None \
                else np.random.normal(0, INIT_WEIGHT_STD, size=(d,))
            self.x = np.tile(x0, (n, 1)).T.copy()
            self.x_estimate = np.copy(self.x)
            self.x_hat = np.copy(self.x)
        per, indices = self.split_indices(y, num_samples)
        if len(np.unique(y)) > 2:
            y[y < 5] = -1
            y[y >= 5] = 1
        losses = np.zeros(p.num_epoch + 1)
        losses[0] = self.loss(A, y)
        every = max(1, int(per / LOSS_PER_EPOCH))
        all_losses = np.zeros(int(per * p.num_epoch / every) + 1)
        W, eye = self.W, np.eye(n)
        bits = self.bits_per_node_iteration(d)
        t_start = time.time()
        sparse_rows = hasattr(A, "tocsr")
        for epoch in range(p.num_epoch):
            stop = False
            for it in range(per):
                t = epoch * per + it
                if t % every == 0:
                    loss = self.loss(A, y)
                    all_losses[t // every] = loss
                    if self.verbose:
                        print("{} t {} epoch {} iter {} loss {} elapsed {:.1f}s".format(p, t, epoch, it, loss,
                                                                                        time.time() - t_start))
                    if not np.isfinite(loss):
                        stop = True
                        break
                lr = self.lr(epoch, it, per, d)
                rows = np.array([rs.choice(indices[m]) for m in range(n)])
                a = A[rows]
                if sparse_rows:
                    a = np.asarray(a.todense())
                ys = y[rows]
                margins = np.einsum("md,dm->m", a, self.x)
                coef = ys * sigmoid(-ys * margins)
                minus_grad = (a * coef[:, None]).T
                if p.regularizer:
                    minus_grad = minus_grad - p.regularizer * self.x
                x_plus = lr * minus_grad
                if p.method == "plain":
                    self.x = (self.x + x_plus) @ W
                elif p.method == "choco":
                    x_plus = x_plus + self.x
                    self.x = x_plus + p.consensus_lr * (self.x_hat @ (W - eye))
                    self.x_hat = self.x_hat + self.quantize(self.x - self.x_hat, rs)
                elif p.method == "dcd-psgd":
                    x_plus = x_plus + self.x @ W
                    self.x = self.x + self.quantize(x_plus - self.x, rs)
                else:  # ecd-psgd
                    x_plus = x_plus + self.x_hat @ W
                    z = (1 - 0.5 * (t + 1)) * self.x + 0.5 * (t + 1) * x_plus
                    q = self.quantize(z, rs)
                    self.x = np.copy(x_plus)
                    self.x_hat = (1 - 2.0 / (t + 1)) * self.x_hat + 2.0 / (t + 1) * q
                self.transmitted_bits += bits * n
                self.update_estimate(t)
            if stop:
                break
            losses[epoch + 1] = self.loss(A, y)
            if self.verbose:
                print("epoch {}: loss {} score {}".format(epoch, losses[epoch + 1], self.score(A, y)))
            if not np.isfinite(losses[epoch + 1]):
                break
        self.train_seconds = time.time() - t_start
        return losses, all_losses

    # ---- GPU path --------------------------------------------------------------------------------------
    def _quantize_torch(self, x, gen):
        import torch

        p, q = self.params, self.params.quantization
        if q == "full":
            return x
        d, n = x.shape
        if q in ("qsgd-biased", "qsgd-unbiased"):
            s = p.num_levels
            norm = x.norm(dim=0, keepdim=True)
            safe = torch.where(norm > 0, norm, torch.ones_like(norm))
            level = s * x.abs() / safe
            low = level.floor()
            new = low + (torch.rand(x.shape, generator=gen, device=x.device, dtype=x.dtype) < (level - low)).to(x.dtype)
            scale = 1.0 / (min(d / s ** 2, np.sqrt(d) / s) + 1.0) if q == "qsgd-biased" else 1.0
            return torch.where(norm > 0, scale * torch.sign(x) * norm * new / s, torch.zeros_like(x))
        k = p.coordinates_to_keep
        out = torch.zeros_like(x)
        if q == "top":
            idx = x.abs().topk(k, dim=0).indices
        else:
            idx = torch.rand(x.shape, generator=gen, device=x.device).topk(k, dim=0).indices
        out.scatter_(0, idx, x.gather(0, idx))
        return d / k * out if q == "random-unbiased" else out

    def _fit_torch(self, A, y_init):
        """Same recurrences with the state, the data and the compressor on the device.  Rows are
        sampled with the host RNG (drawn one epoch ahead), compressor randomness comes from a
        seeded device generator."""
        import torch

        p = self.params
        dev = torch.device(self.device)
        dt = torch.float64
        y = np.copy(y_init)
        num_samples, d = A.shape
        n = p.n_cores
        rs = np.random.RandomState(p.random_seed)
        gen = torch.Generator(device=dev)
        gen.manual_seed(int(p.random_seed or 0))
        x0 = np.random.RandomState(p.random_seed).normal(0, INIT_WEIGHT_STD, size=(d,))
        per, indices = self.split_indices(y, num_samples)
        if len(np.unique(y)) > 2:
            y[y < 5] = -1
            y[y >= 5] = 1
        At = torch.as_tensor(np.asarray(A), dtype=dt, device=dev)
        yt = torch.as_tensor(y, dtype=dt, device=dev)
        x = torch.as_tensor(np.tile(x0, (n, 1)).T.copy(), dtype=dt, device=dev)
        x_hat, x_est = x.clone(), x.clone()
        W = torch.as_tensor(self.W, dtype=dt, device=dev)
        WmI = W - torch.eye(n, dtype=dt, device=dev)
        lam = p.regularizer or 0.0

        A32 = y32 = None
        if dev.type == "cuda" and d % 4 == 0:
            try:  # hand-written full-data loss kernel (fp32 features, fp64 accumulation)
                from ..ops.logreg import logreg_loss

                A32, y32 = At.float().contiguous(), yt.float().contiguous()
            except Exception:
                A32 = None

        def loss_of(xe):
            xm = xe.mean(dim=1)
            if A32 is not None:
                return logreg_loss(A32, y32, xm.contiguous(), lam)
            out = torch.nn.functional.softplus(-yt * (At @ xm)).sum() / num_samples
            return float(out + lam * (xm * xm).sum() / 2)

        losses = np.zeros(p.num_epoch + 1)
        losses[0] = loss_of(x_est)
        every = max(1, int(per / LOSS_PER_EPOCH))
        all_losses = np.zeros(int(per * p.num_epoch / every) + 1)
        t_start = time.time()
        # hand-written path: the whole iteration (every node's stochastic gradient, the gossip step in
        # matrix form and the column compressor) is ONE kernel launch
        fused = None
        if A32 is not None and p.estimate == "final" and not getattr(self, "force_torch_ops", False):
            from ..ops.logreg import LogregIterator, iter_supported

            if iter_supported(n, d):
                fused = LogregIterator(A32, y32, W, x.t().contiguous(), p.method, p.quantization,
                                       k=p.coordinates_to_keep, levels=p.num_levels, lam=lam,
                                       gamma=p.consensus_lr or 0.0, seed=int(p.random_seed or 0))
        for epoch in range(p.num_epoch):
            rows_epoch = torch.as_tensor(
                np.stack([[rs.choice(indices[m]) for m in range(n)] for _ in range(per)]), device=dev)
            if fused is not None:
                for it in range(per):
                    t = epoch * per + it
                    if t % every == 0:
                        all_losses[t // every] = loss_of(fused.state[0].t())
                    fused.step(rows_epoch[it], self.lr(epoch, it, per, d), t)
                x, x_hat = fused.state[0].t(), fused.state[1].t()
                x_est = x
                losses[epoch + 1] = loss_of(x_est)
                if not np.isfinite(losses[epoch + 1]):
                    break
                continue
            for it in range(per):
                t = epoch * per + it
                if t % every == 0:
                    all_losses[t // every] = loss_of(x_est)
                lr = self.lr(epoch, it, per, d)
                rows = rows_epoch[it]
                a, ys = At[rows], yt[rows]
                margins = (a * x.t()).sum(dim=1)
                coef = ys * torch.sigmoid(-ys * margins)
                x_plus = lr * ((a * coef[:, None]).t() - lam * x)
                if p.method == "plain":
                    x = (x + x_plus) @ W
                elif p.method == "choco":
                    x = x_plus + x + p.consensus_lr * (x_hat @ WmI)
                    x_hat = x_hat + self._quantize_torch(x - x_hat, gen)
                elif p.method == "dcd-psgd":
                    x = x + self._quantize_torch(x_plus + x @ W - x, gen)
                else:
                    x_new = x_plus + x_hat @ W
                    z = (1 - 0.5 * (t + 1)) * x + 0.5 * (t + 1) * x_new
                    x_hat = (1 - 2.0 / (t + 1)) * x_hat + 2.0 / (t + 1) * self._quantize_torch(z, gen)
                    x = x_new
                if p.estimate == "final":
                    x_est = x
                else:
                    if p.estimate == "mean":
                        rho = 1 / (t + 1)
                    elif p.estimate == "t+tau":
                        rho = 2 * (t + p.tau) / ((1 + t) * (t + 2 * p.tau))
                    else:
                        rho = 6 * ((t + p.tau) ** 2) / ((1 + t) * (6 * (p.tau ** 2) + t + 6 * p.tau * t + 2 * (t ** 2)))
                    x_est = x_est * (1 - rho) + x * rho
            losses[epoch + 1] = loss_of(x_est)
            if not np.isfinite(losses[epoch + 1]):
                break
        self.x, self.x_hat, self.x_estimate = x.cpu().numpy(), x_hat.cpu().numpy(), x_est.cpu().numpy()
        self.transmitted_bits += self.bits_per_node_iteration(d) * n * per * p.num_epoch
        self.train_seconds = time.time() - t_start
        return losses, all_losses
