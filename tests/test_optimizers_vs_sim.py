"""Every distributed optimizer, run on several Gloo ranks (CPU) with injected gradients,
must reproduce the matrix-form simulator."""
import numpy as np
import pytest
import torch

from chocosgd_b200.config import get_args
from dist_utils import run_ranks


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = torch.nn.Linear(7, 5)
        self.bn1 = torch.nn.BatchNorm1d(5)
        self.fc2 = torch.nn.Linear(5, 3)


def make_model():
    torch.manual_seed(0)
    return Tiny()


def grad_flat(rank, step, seg):
    g = torch.Generator().manual_seed(1000 * rank + step)
    out = torch.zeros(seg.total)
    for sl in seg.slices():
        out[sl] = torch.randn(sl.stop - sl.start, generator=g)
    return out


def conf_for(optimizer, comm_op, topo, n, **kw):
    argv = ["--optimizer", optimizer, "--graph_topology", topo, "--n_mpi_process", str(n), "--lr", "0.05",
            "--momentum_factor", "0.9", "--use_nesterov", "True", "--weight_decay", "0.01",
            "--consensus_stepsize", "0.4", "--backend", "gloo", "--on_cuda", "False", "--gossip_impl", "nccl"]
    if comm_op:
        argv += ["--comm_op", comm_op]
    if comm_op and "compress" in comm_op:
        argv += ["--compress_ratio", "0.7"]
    if comm_op == "quantize_qsgd":
        argv += ["--quantize_level", "4"]
    for k, v in kw.items():
        argv += [f"--{k}", str(v)]
    return get_args(argv)


def worker(rank, world, optimizer, comm_op, topo, steps, extra):
    from chocosgd_b200.optim import define_optimizer
    from chocosgd_b200.parallel.topology import Graph

    conf = conf_for(optimizer, comm_op, topo, world, **extra)
    graph = Graph(topo, world, rank, on_cuda=False)
    model = make_model()
    opt = define_optimizer(conf, model, graph)
    bits = []
    for t in range(steps):
        opt.arena.g.copy_(grad_flat(rank, t, opt.seg))
        bits.append(float(opt.step(epoch=0.5)))
    opt.finalize()
    assert opt.arena.check_bound()
    out = {"x": opt.arena.x.clone().numpy(), "bits": bits}
    if hasattr(opt, "x_hat"):
        out["x_hat"], out["s"] = opt.x_hat.numpy().copy(), opt.s.numpy().copy()
    return out


def simulate(optimizer, comm_op, topo, n, steps, extra):
    from chocosgd_b200.compress.reference import make_codec
    from chocosgd_b200.optim.arena import FlatArena
    from chocosgd_b200.parallel.topology import mixing_matrix
    from chocosgd_b200.sim.matrix_form import Simulator

    conf = conf_for(optimizer, comm_op, topo, n, **extra)
    model = make_model()
    arena = FlatArena(model.named_parameters())
    seg = arena.seg
    wd = [0.0 if "bn" in name else conf.weight_decay for name in seg.names]
    codec = make_codec(seg, comm_op, conf.compress_ratio, conf.quantize_level, None, conf.is_biased, conf.random_k_seed)
    alg = {"sgd": "dpsgd", "parallel_choco_v": "choco", "parallel_choco": "choco"}.get(optimizer, optimizer)
    centralized = optimizer == "sgd" and topo == "complete"
    if optimizer in ("dgc", "ef_sign_sgd") and comm_op is None:
        from chocosgd_b200.compress.reference import SignCodec
        codec = SignCodec(seg)
    sim = Simulator(alg, mixing_matrix(topo, n), arena.x.clone(), seg, codec if comm_op or optimizer == "ef_sign_sgd" else None,
                    lr=conf.lr, consensus_stepsize=conf.consensus_stepsize, weight_decay=wd,
                    momentum=conf.momentum_factor, nesterov=conf.use_nesterov)
    for t in range(steps):
        fn = lambda i, tt, x: grad_flat(i, tt, seg)
        sim.step_centralized(fn) if centralized else sim.step(fn)
    return sim, codec


CASES = [
    ("sgd", None, "complete", 3),
    ("sgd", None, "ring", 4),
    ("parallel_choco_v", "sign", "ring", 3),
    ("parallel_choco_v", "compress_top_k", "ring", 4),
    ("parallel_choco", "compress_random_k", "ring", 4),
    ("parallel_choco_v", "quantize_qsgd", "torus", 9),
    ("parallel_choco_v", "sign", "ring", 2),
    ("dcd_psgd", "compress_top_k", "ring", 3),
    ("dcd_psgd", "sign", "ring", 3),
    ("ecd_psgd", "compress_top_k", "ring", 3),
    ("ecd_psgd", "quantize_qsgd", "ring", 3),
    ("deep_squeeze", "sign", "ring", 4),
    ("deep_squeeze", "compress_top_k", "ring", 3),
    ("dgc", "compress_top_k", "complete", 3),
    ("ef_sign_sgd", None, "complete", 3),
]


def multi_worker(rank, world, cases, steps):
    return [worker(rank, world, o, c, t, steps, {}) for (o, c, t, _) in cases]


@pytest.mark.parametrize("n", sorted({c[3] for c in CASES}))
def test_matches_simulator(n):
    """All cases of one world size share one set of child processes."""
    steps = 5
    cases = [c for c in CASES if c[3] == n]
    res = run_ranks(multi_worker, n, cases, steps)
    for ci, (optimizer, comm_op, topo, _) in enumerate(cases):
        sim, codec = simulate(optimizer, comm_op, topo, n, steps, {})
        tag = f"{optimizer}/{comm_op}/{topo}"
        for r in range(n):
            out = res[r][ci]
            np.testing.assert_allclose(out["x"], sim.x[r].numpy(), rtol=2e-5, atol=2e-6, err_msg=f"{tag} rank {r}")
            if "x_hat" in out:
                np.testing.assert_allclose(out["x_hat"], sim.x_hat[r].numpy(), rtol=2e-5, atol=2e-6, err_msg=tag)
                np.testing.assert_allclose(out["s"], sim.s[r].numpy(), rtol=2e-5, atol=2e-6, err_msg=tag)
        if "choco" in optimizer:
            # the step returns the bits of the previous exchange: nothing on the first step
            assert res[0][ci]["bits"][0] == 0 and res[0][ci]["bits"][1] == codec.n_bits()


def overlap_worker(rank, world):
    a = worker(rank, world, "parallel_choco_v", "sign", "ring", 4, {"overlap_gossip": "True"})
    b = worker(rank, world, "parallel_choco_v", "sign", "ring", 4, {"overlap_gossip": "False"})
    return a, b


def test_choco_overlap_and_blocking_agree():
    res = run_ranks(overlap_worker, 3)
    for r in range(3):
        a, b = res[r]
        np.testing.assert_array_equal(a["x"], b["x"])
        np.testing.assert_array_equal(a["x_hat"], b["x_hat"])


def test_choco_consensus_contracts():
    """Pure gossip (zero gradients, different starting points) reaches the average."""
    from chocosgd_b200.compress.reference import make_codec
    from chocosgd_b200.compress.segments import Segments
    from chocosgd_b200.parallel.topology import mixing_matrix
    from chocosgd_b200.sim.matrix_form import Simulator

    seg = Segments.from_sizes([64, 32])
    x0 = torch.randn(8, seg.total, generator=torch.Generator().manual_seed(0)) * torch.from_numpy(seg.valid_mask()).float()
    sim = Simulator("choco", mixing_matrix("ring", 8), x0, seg, make_codec(seg, "compress_top_k", 0.5), lr=0.0,
                    consensus_stepsize=0.3, identical_init=False)
    e0 = sim.consensus_error()
    mean0 = sim.x.mean(dim=0).clone()
    for _ in range(600):
        sim.step(lambda i, t, x: torch.zeros_like(x))
    assert sim.consensus_error() < 1e-3 * e0
    torch.testing.assert_close(sim.x.mean(dim=0), mean0, atol=1e-4, rtol=1e-4)
