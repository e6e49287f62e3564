"""Aggregators over ``torch.distributed`` (NCCL on GPUs, Gloo on CPU).

This module is the *library* transport: bootstrap, cold-path collectives (metric
averages, model averaging for evaluation, initial weight broadcast) and the
``--gossip_impl nccl`` baseline gossip.  The product gossip path does not pass through
here: it pushes payloads from inside the CUDA kernels into peer-mapped mailboxes
(``parallel/symm.py`` + ``ops/gossip.py``).

API parity with ``dl_code/pcode/utils/communication.py``:
``CentralizedAggregation`` (``:136-227``), ``DecentralizedAggregation`` (``:230-291``),
``EfficientDecentralizedAggregation`` (``:294-352``), ``get_aggregators`` (``:355-365``),
``global_average`` (``:8-20``), ``flatten`` / ``unflatten`` (``:58-85``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


def dist_ready() -> bool:
    return dist.is_available() and dist.is_initialized()


def _comm_device(on_cuda: bool):
    return torch.device("cuda", torch.cuda.current_device()) if on_cuda else torch.device("cpu")


def global_average(total, count, on_cuda=True, group=None) -> float:
    """sum(total over ranks) / sum(count over ranks) with one 2-float all-reduce."""
    if not dist_ready():
        return float(total) / float(count) if count else 0.0
    arr = torch.tensor([float(total), float(count)], dtype=torch.float64, device=_comm_device(on_cuda))
    dist.all_reduce(arr, op=dist.ReduceOp.SUM, group=group)
    s, c = arr.tolist()
    return s / c if c != 0 else 0.0


def elementwise_min(tensor, group=None):
    if dist_ready():
        dist.all_reduce(tensor, op=dist.ReduceOp.MIN, group=group)
    return tensor


def broadcast(tensor, src, group=None):
    if dist_ready():
        dist.broadcast(tensor, src=src, group=group)
    return tensor


def flatten(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    return torch.cat([t.reshape(-1) for t in tensors])


def unflatten(tensors: Sequence[torch.Tensor], flat: torch.Tensor):
    off = 0
    for t in tensors:
        n = t.numel()
        t.data.copy_(flat[off:off + n].view_as(t))
        off += n


def recover_device(data, device=None):
    return data.to(device) if device is not None else data


class Aggregation:
    """Common per-parameter helpers (``communication.py:114-133``)."""

    def _agg(self, data, op, **kw):
        raise NotImplementedError

    def agg_model(self, model, op="avg"):
        """Average the model over the group.  One flat all-reduce instead of the
        reference's one call per parameter tensor."""
        params = [p for p in model.parameters()]
        flat = flatten([p.data for p in params])
        flat = self._agg(flat, op=op)
        unflatten(params, flat)

    def agg_grad(self, model, op="avg"):
        params = [p for p in model.parameters() if p.grad is not None]
        flat = flatten([p.grad.data for p in params])
        flat = self._agg(flat, op=op)
        off = 0
        for p in params:
            p.grad.data.copy_(flat[off:off + p.numel()].view_as(p))
            off += p.numel()


class CentralizedAggregation(Aggregation):
    def __init__(self, rank: int, world: Sequence[int], neighbors_info: Optional[Dict[int, float]] = None, group=None):
        self.rank = rank
        self.ranks = list(neighbors_info.keys()) if neighbors_info else list(world)
        self.world_size = float(len(self.ranks))
        self.group = group  # None = default (whole world) group

    def _agg(self, data, op=None, distributed=True, communication_scheme="all_reduce", async_op=False, **kw):
        if not distributed or not dist_ready() or self.world_size <= 1:
            if communication_scheme == "all_gather":
                return [data]
            return data
        if communication_scheme == "all_reduce":
            if op not in ("avg", "sum"):
                raise NotImplementedError(op)
            if (not async_op and self.group is None and torch.is_tensor(data) and data.is_cuda
                    and data.dtype == torch.float32 and data.is_contiguous()):
                from . import nvls

                ar = nvls.active()   # created once, collectively (main.py): the same answer on every rank
                if ar is not None and data.numel() <= ar.capacity and ar.world == int(self.world_size):
                    out = ar.all_reduce(data.view(-1), average=(op == "avg"))
                    data.view(-1).copy_(out)
                    return data
            req = dist.all_reduce(data, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)
            if async_op:
                return data, req
            return data / self.world_size if op == "avg" else data
        if communication_scheme == "reduce":
            if op != "sum":
                raise NotImplementedError(op)
            req = dist.reduce(data, dst=kw["dst_rank"], op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)
            return (data, req) if async_op else data
        if communication_scheme == "all_gather":
            out = [torch.empty_like(data) for _ in range(int(self.world_size))]
            req = dist.all_gather(out, data, group=self.group, async_op=async_op)
            return (out, req) if async_op else out
        raise NotImplementedError(communication_scheme)

    def complete_wait(self, req):
        req.wait()

    def global_average(self, total, count) -> float:
        on_cuda = dist_ready() and dist.get_backend(self.group) == "nccl"
        return global_average(total, count, on_cuda=on_cuda, group=self.group)


class _Pending:
    def __init__(self, reqs, data):
        self.reqs, self.data = reqs, data

    def wait(self):
        for r in self.reqs:
            r.wait()
        self.reqs = []
        return self.data


class DecentralizedAggregation(Aggregation):
    """Neighbour exchange with point-to-point messages.

    All sends and receives of one exchange are posted as **one batch**
    (``dist.batch_isend_irecv``): with NCCL, unbatched ``isend`` followed by ``irecv`` on
    both ends of an edge (the reference's order, ``communication.py:259-262``) can block
    each other for messages beyond the eager limit."""

    def __init__(self, rank: int, neighbors_info: Dict[int, float], group=None):
        self.rank = rank
        self.neighbors_info = dict(neighbors_info)
        self.neighbor_ranks = [r for r in neighbors_info if r != rank]
        self.world_size = len(neighbors_info)
        self.group = group

    def start(self, data: torch.Tensor) -> _Pending:
        local = {self.rank: data}
        if not self.neighbor_ranks or not dist_ready():
            return _Pending([], local)
        ops = []
        for r in self.neighbor_ranks:
            local[r] = torch.empty_like(data)
        for r in self.neighbor_ranks:
            # graph ranks index the members of ``group``; point-to-point calls address global ranks
            peer = dist.get_global_rank(self.group, r) if self.group is not None else r
            ops.append(dist.P2POp(dist.isend, data, peer, group=self.group))
            ops.append(dist.P2POp(dist.irecv, local[r], peer, group=self.group))
        reqs = dist.batch_isend_irecv(ops)
        return _Pending(reqs, local)

    def _agg(self, data, op, force_wait=True, **kw):
        pending = self.start(data)
        if not force_wait:
            if op != "get_raw_sync_data":
                raise ValueError("deferred completion only returns raw data")
            return pending.reqs, pending.data
        local = pending.wait()
        if op == "avg":
            return sum(local.values()) / self.world_size
        if op == "weighted":
            return sum(t * self.neighbors_info[r] for r, t in local.items())
        if op == "get_raw_sync_data":
            return local
        raise NotImplementedError(op)

    def complete_wait(self, reqs):
        for r in reqs:
            r.wait()


class EfficientDecentralizedAggregation(DecentralizedAggregation):
    """Per-edge transport: one broadcast inside a 2-rank group per directed edge
    (``communication.py:294-352``).  Groups are created collectively, in a global edge
    order, so every rank calls ``new_group`` the same number of times."""

    def __init__(self, rank, neighbors_info, all_edges: Sequence[Sequence[int]]):
        super().__init__(rank, neighbors_info)
        self.edge_group = {}
        for a, b in sorted({tuple(sorted(e)) for e in all_edges}):
            g = dist.new_group([a, b]) if dist_ready() else None
            if rank in (a, b):
                self.edge_group[(a, b)] = g

    def start(self, data):
        local = {self.rank: data}
        reqs = []
        for (a, b), g in sorted(self.edge_group.items()):
            peer = b if a == self.rank else a
            local[peer] = torch.empty_like(data)
            for src in (a, b):  # both directions, same order on both ends
                buf = data if src == self.rank else local[peer]
                reqs.append(dist.broadcast(buf, src=src, group=g, async_op=True))
        return _Pending(reqs, local)


def get_aggregators(cur_rank, world, neighbors_info, aggregator_type, group=None, all_edges=None):
    if "centralized" == aggregator_type:
        return CentralizedAggregation(cur_rank, world, neighbors_info, group)
    if "decentralized" == aggregator_type:
        return DecentralizedAggregation(cur_rank, neighbors_info, group)
    if "efficient_decentralized" == aggregator_type:
        return EfficientDecentralizedAggregation(cur_rank, neighbors_info, all_edges)
    raise NotImplementedError(aggregator_type)


def consistent_model(model, on_cuda=True, group=None):
    """Give every rank rank-0's initial weights: one flat broadcast (the reference zeroes
    the other ranks and all-reduces every tensor, ``dl_code/pcode/create_model.py:92-102``)."""
    if not dist_ready() or dist.get_world_size(group) <= 1:
        return
    tensors = [p.data for p in model.parameters()] + [b.data for b in model.buffers() if b.dtype.is_floating_point]
    flat = flatten(tensors)
    dist.broadcast(flat, src=0, group=group)
    unflatten(tensors, flat)
