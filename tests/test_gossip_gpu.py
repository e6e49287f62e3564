"""The fused CUDA gossip kernels against the matrix-form simulator, with all logical ranks
on one GPU (loopback): same kernels, same flags / parities / payload layouts as the
multi-GPU path, minus NVLink."""
import numpy as np
import pytest
import torch

from chocosgd_b200.compress.reference import make_codec
from chocosgd_b200.compress.segments import Segments
from chocosgd_b200.parallel.topology import mixing_matrix
from chocosgd_b200.sim.matrix_form import Simulator

pytestmark = pytest.mark.gpu

SIZES = [10, 64, 33, 1, 1500, 31, 4100, 257]


def _grad(seg, n, t, scale=1.0):
    g = torch.Generator().manual_seed(100 + t)
    out = torch.zeros(n, seg.total)
    for sl in seg.slices():
        out[:, sl] = torch.randn(n, sl.stop - sl.start, generator=g) * scale
    return out


def _x0(seg):
    g = torch.Generator().manual_seed(7)
    x = torch.zeros(seg.total)
    for sl in seg.slices():
        x[sl] = torch.randn(sl.stop - sl.start, generator=g)
    return x


def _run(comm_op, topo, n, steps=6, momentum=0.9, nesterov=True, chunk=None, **kw):
    from chocosgd_b200.ops.gossip import LoopbackWorld

    seg = Segments.from_sizes(SIZES)
    wd = [0.0 if i % 3 == 0 else 1e-2 for i in range(seg.n_segments)]
    w = mixing_matrix(topo, n)
    x0 = _x0(seg)
    codec = make_codec(seg, comm_op, kw.get("compress_ratio"), kw.get("quantize_level"), kw.get("qsgd_levels"),
                       kw.get("is_biased", False), 1234)
    sim = Simulator("choco", w, x0, seg, codec, lr=0.05, consensus_stepsize=0.4, weight_decay=wd,
                    momentum=momentum, nesterov=nesterov)
    world = LoopbackWorld(w, seg, x0, comm_op, wd, device="cuda", chunk_elems=chunk, **kw)
    for t in range(steps):
        g = _grad(seg, n, t)
        sim.step(lambda i, tt, x: g[i])
        world.step(g, 0.05, momentum, 0.4, nesterov)
    world.flush()
    torch.cuda.synchronize()
    assert world.engine.step_index() == steps
    return sim, world, seg


@pytest.mark.parametrize("topo,n", [("ring", 1), ("ring", 2), ("ring", 4), ("ring", 8), ("complete", 4), ("complete", 8),
                                    ("torus", 9)])
def test_sign_matches_simulator(topo, n):
    sim, world, seg = _run("sign", topo, n)
    torch.testing.assert_close(world.x.cpu(), sim.x, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(world.x_hat.cpu(), sim.x_hat, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(world.s.cpu(), sim.s, rtol=2e-5, atol=2e-6)
    pad = ~torch.from_numpy(seg.valid_mask())
    assert world.x.cpu()[:, pad].abs().sum() == 0 and world.x_hat.cpu()[:, pad].abs().sum() == 0
    assert world.g.abs().sum() == 0  # the kernel consumes (zeroes) the gradient


def test_sign_multi_chunk_segments_and_no_momentum():
    sim, world, _ = _run("sign", "ring", 3, momentum=0.0, nesterov=False, chunk=1024)
    torch.testing.assert_close(world.x.cpu(), sim.x, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(world.s.cpu(), sim.s, rtol=2e-5, atol=2e-6)


def test_sign_is_bitwise_reproducible():
    _, a, _ = _run("sign", "ring", 4)
    _, b, _ = _run("sign", "ring", 4)
    assert torch.equal(a.x, b.x) and torch.equal(a.x_hat, b.x_hat) and torch.equal(a.s, b.s)


@pytest.mark.parametrize("coop", [True, False])   # one cooperative kernel per step / chain of kernels
@pytest.mark.parametrize("topo,n", [("ring", 1), ("ring", 4), ("complete", 5)])
def test_topk_matches_simulator(topo, n, coop):
    sim, world, _ = _run("compress_top_k", topo, n, compress_ratio=0.9, coop=coop)
    assert world.engine.coop == coop and (world.engine.launches_per_step == 1) == coop
    torch.testing.assert_close(world.x.cpu(), sim.x, rtol=2e-5, atol=2e-6)
    # same coordinates selected: x_hat has the same support
    assert torch.equal(world.x_hat.cpu() != 0, sim.x_hat != 0)
    torch.testing.assert_close(world.x_hat.cpu(), sim.x_hat, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(world.s.cpu(), sim.s, rtol=2e-5, atol=2e-6)


def test_topk_with_ties_takes_lowest_indices():
    """Identical magnitudes everywhere: the k lowest indices of every tensor are selected."""
    from chocosgd_b200.ops.gossip import LoopbackWorld

    seg = Segments.from_sizes([100, 3000])
    x0 = torch.zeros(seg.total)
    for sl in seg.slices():
        x0[sl] = 1.0
    world = LoopbackWorld(mixing_matrix("ring", 1), seg, x0, "compress_top_k", 0.0, device="cuda", compress_ratio=0.9)
    world.step(torch.zeros(1, seg.total), 0.0, 0.0, 0.5, False)
    world.flush()
    xh = world.x_hat.cpu()[0]
    for sl, k in zip(seg.slices(), seg.keep_counts(0.9)):
        nz = (xh[sl] != 0).nonzero().view(-1)
        assert nz.tolist() == list(range(k))


@pytest.mark.parametrize("coop", [True, False])
@pytest.mark.parametrize("topo,n", [("ring", 1), ("ring", 4)])
def test_randomk_matches_simulator(topo, n, coop):
    sim, world, _ = _run("compress_random_k", topo, n, compress_ratio=0.8, coop=coop)
    assert world.engine.coop == coop and (world.engine.launches_per_step == 1) == coop
    torch.testing.assert_close(world.x.cpu(), sim.x, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(world.x_hat.cpu(), sim.x_hat, rtol=2e-5, atol=2e-6)
    torch.testing.assert_close(world.s.cpu(), sim.s, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("kw", [{"quantize_level": 4}, {"qsgd_levels": 16, "is_biased": True}])
def test_qsgd_matches_simulator(kw):
    sim, world, _ = _run("quantize_qsgd", "ring", 4, **kw)
    # a level can flip where s|d|/norm sits on a rounding boundary (norms are summed in a
    # different order): allow a handful of elements to differ by one quantization step
    for a, b in ((world.x.cpu(), sim.x), (world.x_hat.cpu(), sim.x_hat), (world.s.cpu(), sim.s)):
        bad = ~torch.isclose(a, b, rtol=1e-4, atol=1e-5)
        assert bad.float().mean() < 2e-3, float(bad.float().mean())


@pytest.mark.parametrize("comm_op", ["compress_top_k", "compress_random_k"])
def test_cooperative_step_equals_the_kernel_chain_bitwise(comm_op):
    """Multi-chunk tensors, several steps: same x, x_hat, s from the one-kernel step and the chain."""
    a = _run(comm_op, "ring", 3, chunk=1024, compress_ratio=0.9, coop=True)[1]
    b = _run(comm_op, "ring", 3, chunk=1024, compress_ratio=0.9, coop=False)[1]
    assert a.engine.coop and not b.engine.coop
    assert torch.equal(a.x, b.x) and torch.equal(a.x_hat, b.x_hat) and torch.equal(a.s, b.s)


def test_cooperative_step_times_out_without_hanging():
    """The one-kernel top-k step with a neighbour that never publishes: the flag wait runs out, every CTA
    leaves at the next grid barrier, the host raises, the context stays usable."""
    from chocosgd_b200.ops.gossip import ChocoEngine, RankBuffers
    from chocosgd_b200.parallel.symm import LoopbackMailbox
    from chocosgd_b200.utils.error_handler import GossipTimeout

    seg = Segments.from_sizes([5000, 40])
    dev = torch.device("cuda")
    mk = lambda: torch.zeros(seg.total, device=dev)
    bufs = {0: RankBuffers(torch.ones(seg.total, device=dev), mk(), mk(), mk(), mk())}
    eng = ChocoEngine([0], bufs, {0: {0: 0.5, 1: 0.5}}, seg, [0.0, 0.0], "compress_top_k",
                      lambda pw: LoopbackMailbox({0: [1], 1: [0]}, pw, dev), dev, wait_budget_ms=20.0,
                      compress_ratio=0.9, chunk_elems=1024, coop=True)
    assert eng.coop and eng.coop_grid > 1
    eng.set_hyper(0.1, 0.0, 0.5, False)
    eng.launch_step()
    eng.check()
    eng.launch_step()  # waits for rank 1's payload of step 0, which never comes
    torch.cuda.synchronize()
    with pytest.raises(GossipTimeout) as ei:
        eng.check()
    assert ei.value.peer == 1 and ei.value.step == 0
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0


def test_wait_times_out_without_hanging():
    """A neighbour that never publishes: the bounded wait expires, the kernel returns and the
    host raises; the context stays usable."""
    from chocosgd_b200.ops.gossip import ChocoEngine, RankBuffers
    from chocosgd_b200.parallel.symm import LoopbackMailbox
    from chocosgd_b200.utils.error_handler import GossipTimeout

    seg = Segments.from_sizes([100, 40])
    dev = torch.device("cuda")
    mk = lambda: torch.zeros(seg.total, device=dev)
    bufs = {0: RankBuffers(mk(), mk(), mk(), mk(), mk())}
    nbh = {0: {0: 0.5, 1: 0.5}}
    eng = ChocoEngine([0], bufs, nbh, seg, [0.0, 0.0], "sign",
                      lambda pw: LoopbackMailbox({0: [1], 1: [0]}, pw, dev), dev, wait_budget_ms=20.0)
    eng.set_hyper(0.1, 0.0, 0.5, False)
    eng.launch_step()  # step 0: nothing to wait for
    eng.check()
    eng.launch_step()  # step 1 waits for rank 1's payload of step 0, which never comes
    torch.cuda.synchronize()
    with pytest.raises(GossipTimeout) as ei:
        eng.check()
    assert ei.value.peer == 1 and ei.value.step == 0
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0  # context still alive


@pytest.mark.parametrize("n,chunk", [(2, None), (4, 1024), (8, 1024), (3, 1024)])
def test_fused_allreduce_sgd_matches_centralized_simulator(n, chunk):
    """Two-shot all-reduce + momentum-SGD in one (cooperative, all ranks in one launch) kernel
    against the averaged-gradient simulator; replicas must stay bit-identical."""
    from chocosgd_b200.ops.gossip import LoopbackWorld

    seg = Segments.from_sizes(SIZES)
    wd = [0.0 if i % 3 == 0 else 1e-2 for i in range(seg.n_segments)]
    w = mixing_matrix("complete", n)
    x0 = _x0(seg)
    sim = Simulator("choco", w, x0, seg, None, lr=0.05, consensus_stepsize=0.0, weight_decay=wd, momentum=0.9,
                    nesterov=True)
    world = LoopbackWorld(w, seg, x0, "allreduce", wd, device="cuda", chunk_elems=chunk)
    for t in range(5):
        g = _grad(seg, n, t)
        sim.step_centralized(lambda i, tt, x: g[i])
        world.step(g, 0.05, 0.9, 0.0, True)
    world.flush()
    torch.cuda.synchronize()
    assert world.engine.step_index() == 5
    torch.testing.assert_close(world.x.cpu(), sim.x, rtol=2e-5, atol=2e-6)
    for i in range(1, n):
        assert torch.equal(world.x[i], world.x[0])
    assert world.g.abs().sum() == 0


def test_fused_allreduce_times_out_without_hanging():
    """A peer that never takes part: both bounded waits expire and the host raises."""
    from chocosgd_b200.ops.gossip import ChocoEngine, RankBuffers
    from chocosgd_b200.parallel.symm import LoopbackMailbox
    from chocosgd_b200.utils.error_handler import GossipTimeout

    seg = Segments.from_sizes([100, 40])
    dev = torch.device("cuda")
    mk = lambda: torch.zeros(seg.total, device=dev)
    bufs = {0: RankBuffers(mk(), mk(), mk(), mk(), mk())}
    eng = ChocoEngine([0], bufs, {0: {0: 0.5, 1: 0.5}}, seg, [0.0, 0.0], "allreduce",
                      lambda pw: LoopbackMailbox({0: [1], 1: [0]}, pw, dev), dev, wait_budget_ms=20.0)
    eng.set_hyper(0.1, 0.0, 0.0, False)
    eng.launch_allreduce_sgd()
    torch.cuda.synchronize()
    with pytest.raises(GossipTimeout) as ei:
        eng.check()
    assert ei.value.peer == 1
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0  # context still alive


def test_fused_sgd_and_clip():
    from chocosgd_b200.ops.gossip import ChocoEngine, RankBuffers
    from chocosgd_b200.parallel.symm import LoopbackMailbox
    from chocosgd_b200.ops.sgd import grad_clip_

    seg = Segments.from_sizes(SIZES)
    dev = torch.device("cuda")
    wd = [1e-2] * seg.n_segments
    x = _x0(seg).to(dev)
    g0 = _grad(seg, 1, 0)[0].to(dev)
    xr, m_ref = x.clone(), None
    bufs = {0: RankBuffers(x, torch.zeros_like(x), torch.zeros_like(x), torch.zeros_like(x), torch.zeros_like(x))}
    eng = ChocoEngine([0], bufs, {0: {0: 1.0}}, seg, wd, None, lambda pw: LoopbackMailbox({0: []}, pw, dev), dev)
    valid = torch.from_numpy(seg.valid_mask()).to(dev)
    for t in range(3):
        g = _grad(seg, 1, t)[0].to(dev)
        bufs[0].g.copy_(g)
        norm = grad_clip_(eng, 0.4)[0]
        coef = min(1.0, 0.4 / (float(g.norm()) + 1e-6))
        assert abs(float(norm) - float(g.norm())) < 1e-3 * float(g.norm())
        eng.set_hyper(0.1, 0.9, 0.0, True)
        eng.launch_sgd_only()
        d = g * coef + 1e-2 * xr * valid
        m_ref = d.clone() if m_ref is None else 0.9 * m_ref + d
        xr = xr - 0.1 * (d + 0.9 * m_ref)
    torch.testing.assert_close(x, xr, rtol=2e-5, atol=2e-6)
    assert bufs[0].g.abs().sum() == 0


def test_sign_pack_kernel_matches_cpu_twin():
    from chocosgd_b200.ops.compress import sign_pack, sign_unpack

    for n in (1, 31, 32, 33, 1000, 100003):
        x = torch.randn(n)
        x[0] = 0.0
        wc, wg = sign_pack(x), sign_pack(x.cuda())
        assert torch.equal(wc, wg.cpu())
        assert torch.equal(sign_unpack(wg, n, 0.5).cpu(), torch.where(x < 0, -0.5, 0.5))


def test_logreg_loss_kernel_and_device_simulator():
    import numpy as np

    from chocosgd_b200.convex import LogisticDecentralizedSGD, Parameters
    from chocosgd_b200.convex.data import synthetic_logistic
    from chocosgd_b200.ops.logreg import logreg_loss

    A, y = synthetic_logistic(3000, 200, seed=0)
    x = np.random.RandomState(1).randn(200) * 0.3
    z = -y * (A @ x)
    ref = np.logaddexp(0, z).mean() + 0.5 * 1e-3 * (x * x).sum()
    got = logreg_loss(torch.tensor(A, dtype=torch.float32).cuda(), torch.tensor(y, dtype=torch.float32).cuda(),
                      torch.tensor(x).cuda(), 1e-3)
    assert abs(got - ref) < 1e-5 * abs(ref)
    kw = dict(num_epoch=1, lr_type="decay", initial_lr=0.1, tau=200.0, regularizer=1 / 3000, n_cores=9, topology="ring",
              method="choco", quantization="top", coordinates_to_keep=4, consensus_lr=0.04, distribute_data=True,
              split_data_strategy="random", random_seed=1, split_data_random_seed=1)
    cpu = LogisticDecentralizedSGD(Parameters(**kw))
    gpu = LogisticDecentralizedSGD(Parameters(**kw), device="cuda")
    lc, _ = cpu.fit(A, y)
    lg, _ = gpu.fit(A, y)
    assert abs(lc[-1] - lg[-1]) < 2e-3 * lc[-1]  # same rows sampled, same top-k: same trajectory up to rounding
