"""Host-side failure detection and the policy after a peer is lost.

The reference only has a process-group timeout and ``MPI_Abort`` on divergence
(``dl_code/main.py:39``, ``dl_code/pcode/utils/error_handler.py:37-47``).  Here:

* ``Heartbeat`` - every rank publishes its step in a key-value store between steps (never while
  a kernel or collective of its own is in flight) and reads its neighbours' keys; a rank that
  leaves writes ``-1`` first, a rank that died is noticed when its key stops advancing for
  ``stale_after_s`` seconds;
* on the device, every wait on a peer flag is bounded and ends in a status word
  (``utils.error_handler.GossipTimeout``), so a vanished peer can never hang a GPU;
* ``survivor_graph`` - drop the lost nodes' edges and re-normalise the mixing matrix with
  Metropolis weights; CHOCO's ``x_hat`` / ``s`` are then re-zeroed consistently on all survivors
  (``ChocoSGD.reset_consensus_state``), which is valid because they are re-built from the
  exchanged differences."""
from __future__ import annotations

import time
from typing import Dict, List, Optional

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
        """Publish this rank's step, raise ``PeerLost`` if a neighbour left or went silent."""
        self.beat(step)
        lost = self.lost_peers()
        if lost:
            raise PeerLost(lost)


def survivor_graph(graph, lost):
    """Graph over the surviving ranks (renumbered) with Metropolis weights."""
    return graph.without(lost)
