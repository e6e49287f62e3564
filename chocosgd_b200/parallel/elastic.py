"""Host-side failure detection and recovery after a peer is lost.

The reference only has a process-group timeout and ``MPI_Abort`` on divergence
(``dl_code/main.py:39``, ``dl_code/pcode/utils/error_handler.py:37-47``): a lost rank ends the run.
Here a run can continue on the survivors:

* ``Heartbeat`` - every rank publishes its step in the rendezvous key-value store between steps
  (never while a kernel or collective of its own is in flight) and reads the others' keys; a rank
  that leaves writes ``-1`` first, a rank that died is noticed when its key stops advancing for
  ``stale_after_s`` seconds;
* on the device every wait on a peer flag is bounded and ends in a status word
  (``utils.error_handler.GossipTimeout``), so a vanished peer can never hang a GPU; the trainer
  turns such a timeout into a membership check;
* ``Membership.agree`` - the survivors publish the set of ranks each of them saw leave and take the
  union, so all of them rebuild the same graph even when only the neighbours of the lost rank
  noticed it;
* ``Membership.regroup`` - a process group over the survivors and the survivor graph: the lost
  nodes' edges dropped, the mixing matrix re-normalised with Metropolis weights, ranks renumbered;
* ``rebuild_optimizer`` - a fresh optimizer of the same kind on the new graph and group (new
  mailboxes, new engine).  The parameters and the momentum carry over; what an algorithm keeps
  about its neighbours is reset the way it is initialised (CHOCO: ``x_hat = s = 0``; DCD / ECD:
  replicas = own parameters; error memories = 0), which is consistent because every survivor does
  it at the same step.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

from ..utils.error_handler import PeerLost


class Heartbeat:
    def __init__(self, store, rank: int, peers: List[int], prefix: str = "hb", stale_after_s: Optional[float] = None):
        self.store, self.rank, self.peers, self.prefix = store, rank, list(peers), prefix
        self.stale_after_s = stale_after_s
        self._seen: Dict[int, tuple] = {}
        self.beat(0)

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def beat(self, step: int):
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self):
        """Announce an orderly exit (call between steps)."""
        self.store.set(self._key(self.rank), "-1")

    def lost_peers(self) -> List[int]:
        now, lost = time.time(), []
        for r in self.peers:
            try:
                v = int(self.store.get(self._key(r)).decode())
            except Exception:
                continue
            if v < 0:
                lost.append(r)
                continue
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)
            elif self.stale_after_s is not None and now - last[1] > self.stale_after_s:
                lost.append(r)
        return lost

    def check(self, step: int):
        """Publish this rank's step, raise ``PeerLost`` if a watched rank left or went silent."""
        self.beat(step)
        lost = self.lost_peers()
        if lost:
            raise PeerLost(lost)


def survivor_graph(graph, lost):
    """Graph over the surviving ranks (renumbered) with Metropolis weights."""
    return graph.without(lost)


class Membership:
    """Who is still in the run, agreed through the store.

    ``members`` are global ranks (ranks of the default process group).  A generation counter
    separates successive recoveries; all keys live under ``<prefix>/gen<k>/``."""

    def __init__(self, store, rank: int, members: Sequence[int], prefix: str = "member", settle_s: float = 0.5,
                 stale_after_s: Optional[float] = None):
        self.store, self.rank, self.members = store, int(rank), sorted(int(m) for m in members)
        self.prefix, self.settle_s, self.generation = prefix, settle_s, 0
        self.stale_after_s = stale_after_s
        self.heartbeat = self._new_heartbeat()

    def _new_heartbeat(self):
        others = [m for m in self.members if m != self.rank]
        return Heartbeat(self.store, self.rank, others, prefix=f"{self.prefix}/gen{self.generation}/hb",
                         stale_after_s=self.stale_after_s)

    def beat(self, step):
        self.heartbeat.beat(step)

    def leave(self):
        self.heartbeat.leave()

    def lost(self) -> List[int]:
        return self.heartbeat.lost_peers()

    def agree(self, seen_lost: Sequence[int], step: int = 0, timeout_s: float = 30.0):
        """-> ``(lost, resume_step)``: the union of what every survivor saw, and the largest step index
        among the survivors (they noticed the loss at different steps; all resume from that one).
        Each rank publishes ``lost|step``, waits until every member outside the current union has
        published (a rank that never does within ``timeout_s`` is taken as lost too), and repeats
        while the union grows."""
        base = f"{self.prefix}/gen{self.generation}/view"
        union = set(int(r) for r in seen_lost)
        t0 = time.time()
        while True:
            self.store.set(f"{base}/{self.rank}", ",".join(str(r) for r in sorted(union)) + "|" + str(int(step)))
            time.sleep(self.settle_s)
            grown, steps = False, [int(step)]
            for m in self.members:
                if m == self.rank or m in union:
                    continue
                v = None
                while v is None:
                    try:
                        v = self.store.get(f"{base}/{m}").decode() if self._has(f"{base}/{m}") else None
                    except Exception:
                        v = None
                    if v is None:
                        if m in self.heartbeat.lost_peers() or time.time() - t0 > timeout_s:
                            union.add(m)
                            grown = True
                            break
                        time.sleep(0.05)
                if v:
                    lost_csv, their_step = v.split("|")
                    steps.append(int(their_step))
                    theirs = {int(x) for x in lost_csv.split(",") if x}
                    if not theirs <= union:
                        union |= theirs
                        grown = True
            if not grown:
                return sorted(union), max(steps)

    def _has(self, key) -> bool:
        check = getattr(self.store, "check", None)
        if check is None:
            return True
        try:
            return bool(check([key]))
        except Exception:
            return False

    def regroup(self, graph, lost: Sequence[int], backend: Optional[str] = None, timeout_s: float = 60.0):
        """-> ``(survivor graph, process group over the survivors)``.  ``graph`` is the current graph
        (its ranks index ``self.members``); ``lost`` are global ranks."""
        import datetime

        import torch.distributed as dist

        lost_idx = [self.members.index(r) for r in lost if r in self.members]
        new_graph = graph.without(lost_idx)
        self.members = [m for m in self.members if m not in set(lost)]
        self.generation += 1
        group = None
        if dist.is_available() and dist.is_initialized():
            group = dist.new_group(ranks=self.members, backend=backend,
                                   timeout=datetime.timedelta(seconds=timeout_s))
        self.heartbeat = self._new_heartbeat()
        return new_graph, group


def rebuild_optimizer(conf, model, old_opt, graph, group):
    """A fresh optimizer of the same kind on the survivor graph; parameters and momentum carry over."""
    import torch

    from ..optim import define_optimizer

    old_engine = getattr(old_opt, "engine", None)
    momentum = None if old_opt.momentum_buf is None else old_opt.momentum_buf.clone()
    had_momentum = old_opt.local_index > 0 and momentum is not None
    for closable in (old_engine, getattr(old_opt, "_exchange", None), getattr(old_opt, "_gather", None)):
        if closable is not None and closable is not False and hasattr(closable, "close"):
            try:
                closable.close()
            except Exception:
                pass
    lr = old_opt.lr
    new_opt = define_optimizer(conf, model, graph, group)
    for g in new_opt.param_groups:
        g["lr"] = lr
    if had_momentum:
        if new_opt.momentum_buf is None:
            new_opt.momentum_buf = torch.zeros_like(new_opt.arena.x)
        new_opt.momentum_buf.copy_(momentum)
        if getattr(new_opt, "engine", None) is not None:
            new_opt.engine.set_momentum_flags([1] * new_opt.engine.n_local)
    new_opt.local_index = old_opt.local_index
    return new_opt
