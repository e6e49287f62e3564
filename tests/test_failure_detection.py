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
