"""Fused gossip kernels across real GPUs (one process per GPU, payloads pushed over NVLink
into peer-mapped mailboxes) against the matrix-form simulator."""
import os

import numpy as np
import pytest
import torch

from dist_utils import free_port

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = torch.nn.Linear(70, 50)
        self.bn1 = torch.nn.BatchNorm1d(50)
        self.fc2 = torch.nn.Linear(50, 30)


def make_model():
    torch.manual_seed(0)
    return Tiny()


def grad_flat(rank, step, seg):
    g = torch.Generator().manual_seed(1000 * rank + step)
    out = torch.zeros(seg.total)
    for sl in seg.slices():
        out[sl] = torch.randn(sl.stop - sl.start, generator=g)
    return out


def conf_for(comm_op, n):
    from chocosgd_b200.config import get_args

    argv = ["--optimizer", "parallel_choco_v", "--graph_topology", "ring", "--n_mpi_process", str(n), "--lr", "0.05",
            "--momentum_factor", "0.9", "--use_nesterov", "True", "--weight_decay", "0.01",
            "--consensus_stepsize", "0.4", "--gossip_impl", "fused", "--comm_op", comm_op, "--wait_budget_ms", "5000"]
    if "compress" in comm_op:
        argv += ["--compress_ratio", "0.9"]
    if comm_op == "quantize_qsgd":
        argv += ["--quantize_level", "4"]
    return get_args(argv)


def _worker(rank, world, port, comm_ops, steps, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from chocosgd_b200.optim import define_optimizer
        from chocosgd_b200.parallel.topology import Graph

        res = {}
        for comm_op in comm_ops:
            conf = conf_for(comm_op, world)
            graph = Graph("ring", world, rank)
            model = make_model().cuda()
            opt = define_optimizer(conf, model, graph)
            for t in range(steps):
                opt.arena.g.copy_(grad_flat(rank, t, opt.seg))
                opt.step()
            opt.finalize()
            torch.cuda.synchronize()
            res[comm_op] = (opt.arena.x.cpu().numpy(), opt.x_hat.cpu().numpy(), opt.s.cpu().numpy())
            dist.barrier()
            opt.engine.close()
        out[rank] = res
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_fused_choco_over_nvlink_matches_simulator(world):
    if torch.cuda.device_count() < world:
        pytest.skip("not enough GPUs")
    import torch.multiprocessing as mp

    from chocosgd_b200.compress.reference import make_codec
    from chocosgd_b200.optim.arena import FlatArena
    from chocosgd_b200.parallel.topology import mixing_matrix
    from chocosgd_b200.sim.matrix_form import Simulator

    comm_ops = ["sign", "compress_top_k", "compress_random_k", "quantize_qsgd"]
    steps = 6
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, comm_ops, steps, out)) for r in range(world)]
    [p.start() for p in procs]
    [p.join(600) for p in procs]
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for comm_op in comm_ops:
        conf = conf_for(comm_op, world)
        arena = FlatArena(make_model().named_parameters())
        seg = arena.seg
        wd = [0.0 if "bn" in n else conf.weight_decay for n in seg.names]
        codec = make_codec(seg, comm_op, conf.compress_ratio, conf.quantize_level, None, conf.is_biased, conf.random_k_seed)
        sim = Simulator("choco", mixing_matrix("ring", world), arena.x.clone(), seg, codec, lr=conf.lr,
                        consensus_stepsize=conf.consensus_stepsize, weight_decay=wd, momentum=0.9, nesterov=True)
        for t in range(steps):
            sim.step(lambda i, tt, x: grad_flat(i, tt, seg))
        for r in range(world):
            x, xh, s = out[r][comm_op]
            if comm_op == "quantize_qsgd":
                for a, b in ((x, sim.x[r].numpy()), (xh, sim.x_hat[r].numpy()), (s, sim.s[r].numpy())):
                    assert (~np.isclose(a, b, rtol=1e-4, atol=1e-5)).mean() < 5e-3
            else:
                np.testing.assert_allclose(x, sim.x[r].numpy(), rtol=2e-5, atol=2e-6, err_msg=f"{comm_op} x rank {r}")
                np.testing.assert_allclose(xh, sim.x_hat[r].numpy(), rtol=2e-5, atol=2e-6, err_msg=f"{comm_op} x_hat")
                np.testing.assert_allclose(s, sim.s[r].numpy(), rtol=2e-5, atol=2e-6, err_msg=f"{comm_op} s")


OTHER = [("sgd", None, "ring"), ("sgd", None, "complete"), ("dcd_psgd", "compress_top_k", "ring"), ("ecd_psgd", "quantize_qsgd", "ring"),
         ("deep_squeeze", "sign", "ring"), ("dgc", "compress_top_k", "complete"), ("ef_sign_sgd", None, "complete"),
         ("parallel_choco_v", "sign", "ring")]


def conf_other(optimizer, comm_op, topo, n, impl):
    from chocosgd_b200.config import get_args

    argv = ["--optimizer", optimizer, "--graph_topology", topo, "--n_mpi_process", str(n), "--lr", "0.05",
            "--momentum_factor", "0.9", "--use_nesterov", "True", "--weight_decay", "0.01",
            "--consensus_stepsize", "0.4", "--gossip_impl", impl, "--wait_budget_ms", "5000"]
    if comm_op:
        argv += ["--comm_op", comm_op]
    if comm_op and "compress" in comm_op:
        argv += ["--compress_ratio", "0.9"]
    if comm_op == "quantize_qsgd":
        argv += ["--quantize_level", "4"]
    return get_args(argv)


def _worker_other(rank, world, port, steps, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from chocosgd_b200.optim import define_optimizer
        from chocosgd_b200.parallel.exchange import sq_distance
        from chocosgd_b200.parallel.topology import Graph

        res = {}
        for optimizer, comm_op, topo in OTHER:
            xs = {}
            for impl in ("fused", "nccl"):  # mailbox transport vs torch.distributed on the same GPUs
                conf = conf_other(optimizer, comm_op, topo, world, impl)
                if optimizer == "parallel_choco_v" and impl == "fused":
                    continue
                graph = Graph(topo, world, rank)
                model = make_model().cuda()
                opt = define_optimizer(conf, model, graph)
                for t in range(steps):
                    opt.arena.g.copy_(grad_flat(rank, t, opt.seg))
                    opt.step(epoch=0.5)
                opt.finalize()
                torch.cuda.synchronize()
                xs[impl] = opt.arena.x.clone()
                dist.barrier()
            if "fused" in xs:
                d = float(sq_distance(xs["fused"], xs["nccl"]))
                res[f"{optimizer}-{topo}"] = (d, float((xs["nccl"].double() ** 2).sum()))
        out[rank] = res
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_mailbox_transport_equals_library_transport(world):
    """Every other algorithm gives the same parameters whether its payloads travel through the
    peer-mapped mailboxes (in-kernel NVLink stores; for centralized SGD the one-kernel all-reduce +
    update) or through torch.distributed."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = free_port()
    procs = [ctx.Process(target=_worker_other, args=(r, world, port, 5, out)) for r in range(world)]
    [p.start() for p in procs]
    [p.join(600) for p in procs]
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for r in range(world):
        for name, (d, ref) in out[r].items():
            # stochastic rounding levels can flip where s|v|/norm sits on a rounding boundary
            tol = 1e-4 if name.startswith("ecd_psgd") else 1e-10
            assert d <= tol * ref + 1e-12, (name, d, ref)


def _worker_leave(rank, world, port, out):
    """CHOCO-SGD (fused kernels) for three steps; the last rank then leaves between steps (nothing of
    its own in flight, NVLS off, plain peer stores); the others notice it on the host, agree, rebuild
    group / graph / optimizer and take three more steps."""
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    # no device_id: with one, torch creates the survivors' communicator by splitting the default one,
    # which needs the rank that left; without it the new group makes its own rendez-vous (as main.py does)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    from chocosgd_b200.optim import define_optimizer
    from chocosgd_b200.parallel.elastic import Membership, rebuild_optimizer
    from chocosgd_b200.parallel.topology import Graph

    conf = conf_for("sign", world)
    graph = Graph("ring", world, rank)
    model = make_model().cuda()
    opt = define_optimizer(conf, model, graph)
    member = Membership(dist.distributed_c10d._get_default_store(), rank, list(range(world)), settle_s=0.2)
    dist.barrier()
    for t in range(3):
        opt.arena.g.copy_(grad_flat(rank, t, opt.seg))
        opt.step()
        member.beat(t + 1)
    opt.finalize()
    torch.cuda.synchronize()
    dist.barrier()          # every rank has applied the exchange of step 3: nothing is in flight
    if rank == world - 1:
        member.leave()
        out[rank] = {"left": True}
        os._exit(0)
    import time

    t0, lost = time.time(), []
    while not lost and time.time() - t0 < 20:
        time.sleep(0.05)
        lost = member.lost()
    lost, _ = member.agree(lost, step=3)
    x_before = opt.arena.x.clone()
    new_graph, group = member.regroup(graph, lost, backend="nccl")
    opt = rebuild_optimizer(conf, model, opt, new_graph, group)
    for t in range(3, 6):
        opt.arena.g.copy_(grad_flat(rank, t, opt.seg))
        opt.step()
    opt.finalize()
    torch.cuda.synchronize()
    out[rank] = {"lost": lost, "n": new_graph.n_nodes, "x_before": x_before.cpu().numpy(),
                 "x": opt.arena.x.cpu().numpy(), "m": opt.momentum_buf.cpu().numpy()}
    os._exit(0)


@pytest.mark.parametrize("world", [2, 4])
def test_rank_leaves_between_steps_and_the_rest_continue(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    from chocosgd_b200.compress.reference import make_codec
    from chocosgd_b200.optim.arena import FlatArena
    from chocosgd_b200.parallel.topology import Graph
    from chocosgd_b200.sim.matrix_form import Simulator

    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = free_port()
    procs = [ctx.Process(target=_worker_leave, args=(r, world, port, out)) for r in range(world)]
    [p.start() for p in procs]
    [p.join(600) for p in procs]
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    res = dict(out)
    assert res[world - 1] == {"left": True}
    survivors = list(range(world - 1))
    for r in survivors:
        assert res[r]["lost"] == [world - 1] and res[r]["n"] == world - 1
    # the survivors' three steps after the loss follow the CHOCO recurrence on the survivor graph,
    # started from their parameters at the time of the loss with x_hat = s = 0 (momentum carried over)
    conf = conf_for("sign", world)
    arena = FlatArena(make_model().named_parameters())
    seg = arena.seg
    wd = [0.0 if "bn" in n else conf.weight_decay for n in seg.names]
    codec = make_codec(seg, "sign", None, None, None, False, conf.random_k_seed)
    w = Graph("ring", world, 0).without([world - 1]).matrix
    x0 = torch.stack([torch.from_numpy(res[r]["x_before"]) for r in survivors])
    # momentum at the time of the loss = momentum after three steps of the full ring: re-simulate those
    full = Simulator("choco", Graph("ring", world, 0).matrix, arena.x.clone(), seg, codec, lr=conf.lr,
                     consensus_stepsize=conf.consensus_stepsize, weight_decay=wd, momentum=0.9, nesterov=True)
    for t in range(3):
        full.step(lambda i, tt, x: grad_flat(i, tt, seg))
    sim = Simulator("choco", w, x0, seg, codec, lr=conf.lr, consensus_stepsize=conf.consensus_stepsize,
                    weight_decay=wd, momentum=0.9, nesterov=True, identical_init=False)
    sim.local.buf = [full.local.buf[r].clone() for r in survivors]
    for t in range(3, 6):
        sim.step(lambda i, tt, x, t=t: grad_flat(survivors[i], t, seg))   # (the simulator's own clock restarts at 0)
    for i, r in enumerate(survivors):
        np.testing.assert_allclose(res[r]["x"], sim.x[i].numpy(), rtol=1e-4, atol=1e-5, err_msg=f"rank {r}")


def _worker_nvls(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from chocosgd_b200.parallel import nvls

    try:
        res = {}
        ar = nvls.enable(1 << 20)
        if ar is None:
            res["skip"] = nvls.why_not()
        else:
            for n in (4, 1000, 65536 + 12, 1 << 20):
                g = torch.Generator(device="cuda").manual_seed(1000 * rank + n)
                x = torch.randn(n, device="cuda", generator=g)
                ref = x.clone()
                dist.all_reduce(ref)
                for average in (False, True):
                    got = ar.all_reduce(x, average=average).clone()
                    torch.cuda.synchronize()
                    ar.check()
                    want = ref / world if average else ref
                    res[(n, average)] = float((got - want).abs().max() / want.abs().max())
                    # every rank holds the same bits: each element is computed by exactly one rank
                    same = [torch.empty_like(got) for _ in range(world)]
                    dist.all_gather(same, got)
                    res[(n, average, "same")] = all(torch.equal(same[0], s) for s in same)
        out[rank] = res
        torch.cuda.synchronize()
        dist.barrier()
        nvls.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_multimem_allreduce_matches_the_library(world):
    """``multimem.ld_reduce`` / ``multimem.st`` all-reduce kernel against NCCL (skips where the system has
    no NVLink multicast)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    if os.environ.get("NCCL_NVLS_ENABLE", "1") == "0":
        pytest.skip("multicast switched off for this run")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = free_port()
    procs = [ctx.Process(target=_worker_nvls, args=(r, world, port, out)) for r in range(world)]
    [p.start() for p in procs]
    [p.join(300) for p in procs]
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    res = dict(out)
    if "skip" in res[0]:
        pytest.skip("no multicast: " + res[0]["skip"])
    for r in range(world):
        for k, v in res[r].items():
            if len(k) == 3:
                assert v, (r, k)
            else:
                assert v < 1e-5, (r, k, v)
