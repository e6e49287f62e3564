import numpy as np
import pytest

from chocosgd_b200.convex import LogisticDecentralizedSGD, Parameters, mixing_matrix_convex, qsgd_quantize
from chocosgd_b200.convex.data import synthetic_logistic
from chocosgd_b200.convex.experiment import epsilon_final_params, run_experiment


def _params(**kw):
    base = dict(num_epoch=2, lr_type="decay", initial_lr=0.1, tau=100.0, regularizer=1 / 2000, n_cores=9,
                topology="ring", distribute_data=True, split_data_strategy="random", random_seed=1,
                split_data_random_seed=1)
    base.update(kw)
    return Parameters(**base)


def test_parameter_validation():
    with pytest.raises(ValueError):
        Parameters(num_epoch=1, lr_type="nope")
    with pytest.raises(ValueError):
        _params(method="choco", quantization="top", coordinates_to_keep=5)  # consensus_lr missing
    with pytest.raises(ValueError):
        _params(method="dcd-psgd", quantization="top", coordinates_to_keep=5)  # needs an unbiased compressor
    with pytest.raises(ValueError):
        _params(method="plain", quantization="qsgd-unbiased")  # num_levels missing
    p = _params(method="choco", quantization="top", coordinates_to_keep=5, consensus_lr=0.04)
    assert "top5" in str(p)


def test_mixing_matrices():
    w = mixing_matrix_convex("ring", 9)
    assert np.allclose(w.sum(0), 1) and np.allclose(w.sum(1), 1) and np.isclose(w[0, 8], 1 / 3)
    assert np.allclose(mixing_matrix_convex("ring", 2), 0.5)
    assert np.allclose(mixing_matrix_convex("centralized", 4), 0.25)
    assert np.allclose(mixing_matrix_convex("disconnected", 3), np.eye(3))
    assert np.allclose(mixing_matrix_convex("torus", 9).sum(1), 1)


def test_qsgd_is_unbiased():
    rs = np.random.RandomState(0)
    x = rs.randn(50)
    acc = sum(qsgd_quantize(x, 16, False, rs) for _ in range(3000)) / 3000
    assert np.abs(acc - x).max() < 0.05
    assert np.all(qsgd_quantize(np.zeros(5), 4, False, rs) == 0)


@pytest.mark.parametrize("method,kw", [
    ("plain", dict(quantization="full")),
    ("choco", dict(quantization="top", coordinates_to_keep=2, consensus_lr=0.04)),
    ("choco", dict(quantization="random-biased", coordinates_to_keep=5, consensus_lr=0.01)),
    ("choco", dict(quantization="qsgd-biased", num_levels=16, consensus_lr=0.34)),
    ("dcd-psgd", dict(quantization="qsgd-unbiased", num_levels=16)),
])
def test_methods_decrease_the_loss(method, kw):
    A, y = synthetic_logistic(2000, 100, seed=0)
    m = LogisticDecentralizedSGD(_params(method=method, **kw))
    losses, trace = m.fit(A, y)
    assert abs(losses[0] - np.log(2)) < 0.02
    assert losses[-1] < 0.8 * losses[0]
    assert m.score(A, y) > 0.8
    assert len(trace) == 2 * 10 + 1 and m.transmitted_bits > 0


def test_runs_are_reproducible_and_choco_full_equals_exact_gossip():
    A, y = synthetic_logistic(900, 40, seed=1)
    a = LogisticDecentralizedSGD(_params(method="choco", quantization="top", coordinates_to_keep=4, consensus_lr=0.1))
    b = LogisticDecentralizedSGD(_params(method="choco", quantization="top", coordinates_to_keep=4, consensus_lr=0.1))
    la, _ = a.fit(A, y)
    lb, _ = b.fit(A, y)
    assert np.array_equal(la, lb)
    # CHOCO without compression and gamma = 1 mixes the previous iterate exactly (x_hat = x): it differs
    # from plain gossip only by the mixing of the last gradient step, so the curves nearly coincide
    c = LogisticDecentralizedSGD(_params(method="choco", quantization="full", consensus_lr=1.0))
    d = LogisticDecentralizedSGD(_params(method="plain", quantization="full"))
    lc, _ = c.fit(A, y)
    ld, _ = d.fit(A, y)
    assert np.allclose(lc, ld, rtol=1e-2)


def test_bit_model():
    m = LogisticDecentralizedSGD(_params(method="choco", quantization="top", coordinates_to_keep=20, consensus_lr=0.04))
    assert m.bits_per_node_iteration(2000) == (64 + 11) * 2 * 20
    m = LogisticDecentralizedSGD(_params(method="choco", quantization="qsgd-unbiased", num_levels=16, consensus_lr=0.3))
    assert m.bits_per_node_iteration(2000) == (4 + 1) * 2 * 2000
    m = LogisticDecentralizedSGD(_params(method="plain", quantization="full"))
    assert m.bits_per_node_iteration(2000) == 64 * 2 * 2000


def test_experiment_driver(tmp_path):
    A, y = synthetic_logistic(300, 20, seed=2)
    ps = [_params(num_epoch=1, method="plain", quantization="full", name="p"),
          _params(num_epoch=1, method="choco", quantization="top", coordinates_to_keep=2, consensus_lr=0.04, name="c")]
    res = run_experiment(str(tmp_path), (A, y), ps, nproc=2)
    assert len(res) == 2 and (tmp_path / "results.pickle").exists() and (tmp_path / "params.pickle").exists()
    assert len(epsilon_final_params()) == 2 * 5 * 9


def test_convex_bench_tool_runs(capsys):
    import json

    from chocosgd_b200.tools import convex_bench

    convex_bench.main(["--samples", "300", "--features", "100", "--nodes", "3", "--epochs", "1"])
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert [l["method"] for l in lines] == ["choco", "plain"]
    assert all(0.0 < l["final_loss"] < 1.0 for l in lines)
