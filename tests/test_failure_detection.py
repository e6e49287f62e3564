"""Failure detection without any GPU fault: failures are made on the host (a rank that leaves, a
rank that goes silent, a collective that times out) and detected through the store / timeouts."""
import datetime
import os
import time

import numpy as np
import pytest
import torch
import torch.distributed as dist

from dist_utils import free_port, run_ranks


def _leaver(rank, world):
    from chocosgd_b200.parallel.elastic import Heartbeat, survivor_graph
    from chocosgd_b200.parallel.topology import Graph
    from chocosgd_b200.utils.error_handler import PeerLost

    store = dist.distributed_c10d._get_default_store()
    graph = Graph("ring", world, rank, on_cuda=False)
    hb = Heartbeat(store, rank, graph.neighbors())
    dist.barrier()
    for step in range(1, 6):
        if rank == 2 and step == 3:
            hb.leave()  # orderly exit between steps, nothing in flight
            return {"left_at": step}
        time.sleep(0.05)
        try:
            hb.check(step)
        except PeerLost as e:
            g2 = survivor_graph(graph, e.ranks)
            return {"detected_at": step, "lost": e.ranks, "n": g2.n_nodes, "row_sum": float(g2.matrix.sum(1).min()),
                    "new_rank": g2.rank}
    return {"finished": True}


def test_neighbours_detect_a_rank_that_leaves():
    res = run_ranks(_leaver, 4)
    assert res[2] == {"left_at": 3}
    for r in (1, 3):  # ring neighbours of rank 2
        assert res[r]["lost"] == [2] and res[r]["n"] == 3 and abs(res[r]["row_sum"] - 1.0) < 1e-12
    assert res[3]["new_rank"] == 2
    assert res[0] == {"finished": True}  # not a neighbour: keeps going


class _FakeStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode()

    def get(self, k):
        return self.d[k]


def test_silent_peer_is_reported_stale():
    from chocosgd_b200.parallel.elastic import Heartbeat
    from chocosgd_b200.utils.error_handler import PeerLost

    store = _FakeStore()
    a = Heartbeat(store, 0, [1], stale_after_s=0.05)
    b = Heartbeat(store, 1, [0], stale_after_s=0.05)
    a.check(1)
    b.beat(1)
    a.check(2)
    time.sleep(0.12)  # rank 1 stops publishing
    with pytest.raises(PeerLost) as ei:
        a.check(3)
    assert ei.value.ranks == [1]


def _timeout_worker(rank, world):
    # rank 1 never joins the collective: rank 0's all_reduce must end with an error, not hang
    if rank == 1:
        time.sleep(3.0)
        return "absent"
    t = torch.ones(4)
    try:
        pg = dist.new_group([0, 1], timeout=datetime.timedelta(seconds=1)) if False else None
        work = dist.all_reduce(t, async_op=True)
        ok = work.wait(timeout=datetime.timedelta(seconds=1))
        return "completed" if ok else "timed out"
    except Exception as e:
        return "error: " + type(e).__name__


def test_collective_with_absent_rank_times_out():
    res = run_ranks(_timeout_worker, 2)
    assert res[1] == "absent"
    assert res[0] != "completed"


def test_divergence_guard_raises(tmp_path):
    from chocosgd_b200.utils.error_handler import GossipTimeout, PeerLost, TrainingDiverged

    assert issubclass(TrainingDiverged, RuntimeError)
    e = GossipTimeout(1, 3, 7)
    assert (e.status, e.peer, e.step) == (1, 3, 7) and "peer=3" in str(e)
    assert PeerLost([2, 1]).ranks == [1, 2]


def _agree_worker(rank, world):
    """Ranks 0, 1, 3 survive; only ranks 1 and 3 saw rank 2 leave.  All must agree, regroup and
    be able to run a collective on the new group."""
    from chocosgd_b200.parallel.elastic import Membership
    from chocosgd_b200.parallel.topology import Graph

    store = dist.distributed_c10d._get_default_store()
    graph = Graph("ring", world, rank, on_cuda=False)
    m = Membership(store, rank, list(range(world)), settle_s=0.2)
    dist.barrier()
    if rank == 2:
        m.leave()
        return {"left": True}
    time.sleep(0.3)
    seen = m.lost() if rank in (1, 3) else []
    lost, resume = m.agree(seen, step=10 + rank)
    new_graph, group = m.regroup(graph, lost, backend="gloo")
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=group)
    return {"lost": lost, "resume": resume, "n": new_graph.n_nodes, "rank": new_graph.rank, "sum": float(t),
            "members": m.members}


def test_survivors_agree_and_regroup():
    res = run_ranks(_agree_worker, 4)
    assert res[2] == {"left": True}
    for r, new_rank in ((0, 0), (1, 1), (3, 2)):
        assert res[r]["lost"] == [2] and res[r]["resume"] == 13 and res[r]["n"] == 3
        assert res[r]["rank"] == new_rank and res[r]["sum"] == 4.0 and res[r]["members"] == [0, 1, 3]


@pytest.mark.timeout(900)
def test_training_continues_on_the_survivors(tmp_path):
    """Four Gloo ranks train CHOCO-SGD on a ring; rank 2 announces an orderly exit before its third
    step.  The other three notice it through the heartbeat, agree, rebuild graph / group / optimizer
    and finish both epochs, validation and checkpoints included."""
    import json
    import subprocess
    import sys

    root_dir = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ck = tmp_path / "ckpt"
    cmd = [sys.executable, "-m", "chocosgd_b200.run", "--data", "synthetic_cifar10", "--synthetic_size", "256",
           "--arch", "lenet", "--batch_size", "16", "--num_epochs", "2", "--optimizer", "parallel_choco_v",
           "--comm_op", "sign", "--graph_topology", "ring", "--consensus_stepsize", "0.4", "--on_cuda", "False",
           "--backend", "gloo", "--n_mpi_process", "4", "--partition_data", "random", "--lr", "0.05",
           "--lr_schedule_scheme", "custom_multistep", "--lr_change_epochs", "1", "--num_workers", "0",
           "--checkpoint", str(ck), "--summary_freq", "1", "--experiment", "t", "--timestamp", "run1",
           "--elastic", "True", "--heartbeat_every", "1", "--leave_at_step", "2:3", "--train_fast", "False"]
    env = dict(os.environ, PYTHONPATH=root_dir + os.pathsep + os.environ.get("PYTHONPATH", ""), OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, env=env, cwd=root_dir, capture_output=True, text=True, timeout=850)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    root = ck / "synthetic_cifar10" / "lenet" / "t" / "run1"
    for rank in ("0", "1", "3"):
        assert (root / rank / "checkpoint.pth.tar").exists()
        recs = json.load(open(root / rank / "log-1.json"))
        tests = [x for x in recs if x.get("split") == "test" and x.get("type") == "local_model"]
        assert [x["epoch"] for x in tests] == [1.0, 2.0]
    assert "lost ranks [2]: continuing on 3 nodes" in open(root / "0" / "log.txt").read()
    left = json.load(open(root / "2" / "log-1.json"))
    assert max(x["local_index"] for x in left if x.get("split") == "train") == 2
