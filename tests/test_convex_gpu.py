"""The one-kernel-per-iteration device path of the convex simulator (``csrc/logreg.cu``) against the
numpy path: same row draws, deterministic compressors -> same trajectory; stochastic compressors
(own random stream on the device) -> same quality."""
import numpy as np
import pytest
import torch

from chocosgd_b200.convex.data import synthetic_logistic
from chocosgd_b200.convex.logistic import LogisticDecentralizedSGD
from chocosgd_b200.convex.parameters import Parameters

pytestmark = pytest.mark.gpu


def _params(method, quantization, **kw):
    return Parameters(num_epoch=2, lr_type="decay", initial_lr=0.1, tau=64.0, regularizer=1.0 / 720, n_cores=9,
                      topology="ring", method=method, quantization=quantization, estimate="final",
                      distribute_data=True, split_data_strategy="random", split_data_random_seed=3, random_seed=7, **kw)


@pytest.mark.parametrize("method,quantization,kw", [
    ("plain", "full", {}),
    ("choco", "full", {"consensus_lr": 1.0}),
    ("choco", "top", {"coordinates_to_keep": 6, "consensus_lr": 0.04}),
])
def test_device_iteration_kernel_follows_the_numpy_trajectory(method, quantization, kw):
    A, y = synthetic_logistic(720, 64, seed=1)
    p = _params(method, quantization, **kw)
    cpu = LogisticDecentralizedSGD(p)
    l_cpu, tr_cpu = cpu.fit(A, y)
    gpu = LogisticDecentralizedSGD(p, device="cuda")
    l_gpu, tr_gpu = gpu.fit(A, y)
    np.testing.assert_allclose(l_gpu, l_cpu, rtol=2e-6, atol=1e-9)     # fp32 features in the loss kernel
    np.testing.assert_allclose(tr_gpu, tr_cpu, rtol=2e-6, atol=1e-9)
    # (fp32 features against numpy's fp64: entries of x that pass near zero differ by a few 1e-9)
    np.testing.assert_allclose(gpu.x, cpu.x, rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(gpu.x_hat, cpu.x_hat, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("method,quantization,kw", [
    ("choco", "random-biased", {"coordinates_to_keep": 6, "consensus_lr": 0.01}),
    ("choco", "qsgd-biased", {"num_levels": 16, "consensus_lr": 0.34}),
    ("dcd-psgd", "qsgd-unbiased", {"num_levels": 16}),
    # (ECD-PSGD multiplies the compression error by t / 2: with random-k it diverges in numpy too)
    ("ecd-psgd", "qsgd-unbiased", {"num_levels": 256}),
])
def test_device_iteration_kernel_with_stochastic_compressors(method, quantization, kw):
    A, y = synthetic_logistic(720, 64, seed=1)
    p = _params(method, quantization, **kw)
    l_cpu, _ = LogisticDecentralizedSGD(p).fit(A, y)
    gpu = LogisticDecentralizedSGD(p, device="cuda")
    l_gpu, _ = gpu.fit(A, y)
    torch_ops = LogisticDecentralizedSGD(p, device="cuda")
    torch_ops.force_torch_ops = True
    l_ops, _ = torch_ops.fit(A, y)
    assert np.isfinite(l_gpu).all() and l_gpu[-1] < l_gpu[0]
    # different random streams: same regime as the numpy run and as the PyTorch-op device path
    assert abs(l_gpu[-1] - l_cpu[-1]) < 0.15 * abs(l_cpu[0] - l_cpu[-1]) + 2e-2
    assert abs(l_gpu[-1] - l_ops[-1]) < 0.15 * abs(l_ops[0] - l_ops[-1]) + 2e-2
