"""Per-edge transport (one 2-rank group per edge, broadcasts in both directions) against the plain
point-to-point exchange, on Gloo ranks (``dl_code/pcode/utils/communication.py:294-352``)."""
import torch

from dist_utils import run_ranks


def _worker(rank, world):
    from chocosgd_b200.parallel.comm import get_aggregators
    from chocosgd_b200.parallel.topology import Graph

    graph = Graph("ring", world, rank, on_cuda=False)
    nbh = graph.get_neighborhood()
    edges = sorted({tuple(sorted((i, j))) for i in range(world) for j in Graph("ring", world, i, on_cuda=False).get_neighborhood()
                    if j != i})
    eff = get_aggregators(rank, list(range(world)), nbh, "efficient_decentralized", all_edges=edges)
    p2p = get_aggregators(rank, list(range(world)), nbh, "decentralized")
    x = torch.arange(6, dtype=torch.float32) + 10.0 * rank
    got = eff.start(x.clone()).wait()
    ref = p2p.start(x.clone()).wait()
    avg = eff._agg(x.clone(), op="weighted") if hasattr(eff, "_agg") else None
    return {"keys": sorted(got), "same": all(torch.equal(got[k], ref[k]) for k in ref) and sorted(got) == sorted(ref),
            "vals": {k: float(v[0]) for k, v in got.items()},
            "avg": avg.tolist() if torch.is_tensor(avg) else None, "weights": {k: float(w) for k, w in nbh.items()}}


def test_per_edge_groups_deliver_every_neighbours_tensor():
    world = 4
    res = run_ranks(_worker, world)
    for r in range(world):
        nb = sorted({(r - 1) % world, r, (r + 1) % world})
        assert res[r]["keys"] == nb and res[r]["same"]
        assert res[r]["vals"] == {k: 10.0 * k for k in nb}
        if res[r]["avg"] is not None:   # the weighted neighbourhood average built on the exchange
            want = sum(res[r]["weights"][k] * (10.0 * k) for k in nb)
            assert abs(res[r]["avg"][0] - want) < 1e-5
