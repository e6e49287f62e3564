"""Mixing topologies: doubly stochastic matrices ``W`` over ``n`` graph nodes.

On an NVSwitch fabric every peer is one hop away at full bandwidth, so a "ring"
or "torus" is purely a *logical* communication pattern: the graph only selects
which peers a rank exchanges with and with what weight.  A :class:`Graph` is
therefore plain data (matrix + rank); it creates no process groups (the
reference builds one 2-rank group per ring edge, ``dl_code/pcode/utils/topology.py:219-241``).

Matrices reproduce ``dl_code/pcode/utils/topology.py:122-589`` with two
extensions: a ring accepts n = 1 and n = 2 (weights 1/2 for n < 3 as in the
convex code, ``convex_code/logistic.py:31-44``), and ``metropolis`` builds W for
any adjacency matrix.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np


def complete_matrix(n: int) -> np.ndarray:
    return np.full((n, n), 1.0 / n)


def ring_matrix(n: int) -> np.ndarray:
    if n == 1:
        return np.ones((1, 1))
    if n == 2:
        return np.full((2, 2), 0.5)
    w = np.zeros((n, n))
    for i in range(n):
        w[i, i] = w[i, (i + 1) % n] = w[i, (i - 1) % n] = 1.0 / 3.0
    return w


def torus_shape(n: int):
    m = int(np.sqrt(n))
    while n % m != 0:
        m -= 1
    return m, n // m


def torus_matrix(n: int) -> np.ndarray:
    """Periodic 2-d grid m x (n/m), m the largest divisor <= sqrt(n); (A + I) / 5."""
    m, k = torus_shape(n)
    a = np.zeros((n, n))

    def idx(r, c):
        return (r % m) * k + (c % k)

    for r in range(m):
        for c in range(k):
            i = idx(r, c)
            for j in (idx(r + 1, c), idx(r - 1, c), idx(r, c + 1), idx(r, c - 1)):
                if j != i:
                    a[i, j] = 1.0
    a[np.arange(n), np.arange(n)] = 1.0
    return a / 5.0


def expander_matrix(n: int) -> np.ndarray:
    """Cycle plus the chord i <-> i^-1 (mod n); node 0 gets a self loop; all / 3."""

    def modulo_inverse(i, p):
        for j in range(1, p):
            if (j * i) % p == 1:
                return j
        return None

    a = np.zeros((n, n))
    for i in range(n):
        a[i, (i + 1) % n] = 1
        a[(i + 1) % n, i] = 1
    a[0, 0] = 1
    for i in range(1, n):
        inv = modulo_inverse(i, n)
        if inv is not None:
            a[i, inv] = 1
    return a / 3.0


def max_degree_weights(adjacency: np.ndarray) -> np.ndarray:
    """w_ij = 1 / max(deg_i, deg_j) on edges, self weight = remainder.

    Equivalent to the reference's degree-ordered sweep
    (``dl_code/pcode/utils/topology.py:437-445``)."""
    a = (np.asarray(adjacency, dtype=np.float64) > 0).astype(np.float64)
    deg = a.sum(axis=1)
    n = a.shape[0]
    w = np.zeros((n, n))
    for i in range(n):
        for j in range(n):
            if i != j and a[i, j] > 0:
                w[i, j] = 1.0 / max(deg[i], deg[j])
    for i in range(n):
        w[i, i] = 1.0 - w[i].sum()
    return w


def metropolis_matrix(adjacency: np.ndarray) -> np.ndarray:
    """Metropolis-Hastings weights 1 / (1 + max(deg_i, deg_j)) for any undirected graph."""
    a = (np.asarray(adjacency) > 0).astype(np.float64)
    np.fill_diagonal(a, 0)
    deg = a.sum(axis=1)
    n = a.shape[0]
    w = np.zeros((n, n))
    for i in range(n):
        for j in range(n):
            if a[i, j] > 0:
                w[i, j] = 1.0 / (1.0 + max(deg[i], deg[j]))
        w[i, i] = 1.0 - w[i].sum()
    return w


def margulis_matrix(n: int) -> np.ndarray:
    base = int(np.sqrt(n))
    if base * base != n:
        raise ValueError("margulis_expander needs a square number of nodes")
    # nodes are numbered in order of first appearance while the edges are enumerated
    # (the numbering an insertion-ordered graph container gives them).
    index = {}
    edges = []
    for x in range(base):
        for y in range(base):
            for (u, v) in (
                ((x + 2 * y) % base, y),
                ((x + 2 * y + 1) % base, y),
                (x, (y + 2 * x) % base),
                (x, (y + 2 * x + 1) % base),
            ):
                for node in ((x, y), (u, v)):
                    if node not in index:
                        index[node] = len(index)
                edges.append((index[(x, y)], index[(u, v)]))
    a = np.zeros((n, n))
    for i, j in edges:
        a[i, j] = a[j, i] = 1
    return max_degree_weights(a)


def social_matrix(n: int) -> np.ndarray:
    if n != 32:
        raise ValueError("the social graph (Davis southern women) has exactly 32 nodes")
    import networkx

    g = networkx.davis_southern_women_graph()
    a = networkx.to_numpy_array(g)
    return max_degree_weights(a)


def ring_ext_matrix(n: int) -> np.ndarray:
    if not (n > 3 and n % 2 == 0):
        raise ValueError("ring_ext needs an even number of nodes > 3")
    a = np.zeros((n, n))
    for i in range(n):
        a[i, i] = 1
        a[i, (i + 1) % n] = 1
        a[i, (i - 1) % n] = 1
        a[i, (i + n // 2) % n] = 1
    return a / 4.0


def disconnected_matrix(n: int) -> np.ndarray:
    return np.eye(n)


_BUILDERS = {
    "complete": complete_matrix,
    "centralized": complete_matrix,
    "ring": ring_matrix,
    "torus": torus_matrix,
    "expander": expander_matrix,
    "margulis_expander": margulis_matrix,
    "social": social_matrix,
    "ring_ext": ring_ext_matrix,
    "disconnected": disconnected_matrix,
}


def mixing_matrix(topology: str, n: int) -> np.ndarray:
    try:
        return _BUILDERS[topology](n)
    except KeyError:
        raise NotImplementedError(f"unknown topology {topology!r}") from None


def spectral_gap(w: np.ndarray) -> float:
    """rho = 1 - |lambda_2(W)| (second largest eigenvalue modulus)."""
    if w.shape[0] == 1:
        return 1.0
    ev = np.sort(np.abs(np.linalg.eigvals(w)))[::-1]
    return float(1.0 - ev[1])


class Graph:
    """A rank's view of the communication graph.

    Mirrors the attributes the reference's graph classes expose
    (``n_nodes``, ``rank``, ``ranks``, ``world``, ``device``, ``on_cuda``,
    ``scaling``, ``matrix``, ``rho``, ``beta``, ``get_neighborhood``;
    ``dl_code/pcode/utils/topology.py:79-171``)."""

    def __init__(
        self,
        topology: str,
        n_nodes: int,
        rank: int = 0,
        n_sub_process: int = 1,
        world: Optional[Sequence[int]] = None,
        comm_device: str = "cuda",
        on_cuda: bool = True,
        matrix: Optional[np.ndarray] = None,
    ):
        self.topology = topology
        self._n = int(n_nodes)
        self._rank = int(rank)
        self._n_sub = int(n_sub_process)
        if isinstance(world, str):
            world = [int(x) for x in world.split(",")]
        self._world = list(world) if world is not None else list(range(self._n * self._n_sub))
        if len(self._world) < self._n * self._n_sub:
            raise ValueError("--world lists fewer devices than n_mpi_process * n_sub_process")
        self.comm_device = "cpu" if (comm_device in (None, "cpu") or not on_cuda) else "cuda"
        self._on_cuda = bool(on_cuda)
        self._w = np.asarray(matrix if matrix is not None else mixing_matrix(topology, self._n), dtype=np.float64)
        if self._w.shape != (self._n, self._n):
            raise ValueError("mixing matrix has the wrong shape")

    # --- layout -------------------------------------------------------------------------
    @property
    def n_nodes(self) -> int:
        return self._n

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def ranks(self) -> List[int]:
        return list(range(self._n))

    @property
    def world(self) -> List[int]:
        return self._world

    @property
    def device(self) -> List[int]:
        """Device ids owned by this rank (``n_sub_process`` of them)."""
        return self._world[self._rank * self._n_sub:(self._rank + 1) * self._n_sub]

    @property
    def on_cuda(self) -> bool:
        return self._on_cuda

    # --- mixing -------------------------------------------------------------------------
    @property
    def matrix(self) -> np.ndarray:
        return self._w

    @property
    def rho(self) -> float:
        return spectral_gap(self._w)

    @property
    def beta(self) -> float:
        return float(np.linalg.norm(self._w - np.eye(self._n), ord=2))

    @property
    def n_edges(self) -> int:
        a = (self._w != 0).astype(int)
        np.fill_diagonal(a, 0)
        return int(a.sum() // 2)

    def get_neighborhood(self, rank: Optional[int] = None) -> Dict[int, float]:
        """``{peer_rank: w_ij}`` **including the rank itself**."""
        r = self._rank if rank is None else rank
        row = self._w[r]
        return {int(c): float(v) for c, v in enumerate(row) if (v != 0 or c == r)}

    def neighbors(self, rank: Optional[int] = None) -> List[int]:
        r = self._rank if rank is None else rank
        return [j for j in self.get_neighborhood(r) if j != r]

    @property
    def scaling(self) -> int:
        """Neighbourhood size, the ``graph`` LR scale-up factor
        (``dl_code/pcode/utils/topology.py:292-293``)."""
        return len(self.get_neighborhood())

    def get_edges(self):
        """Directed edges (src, dst) leaving and entering this rank."""
        out_edges = [(self._rank, j) for j in self.neighbors()]
        in_edges = [(j, self._rank) for j in self.neighbors()]
        return out_edges, in_edges

    def without(self, lost: Sequence[int]) -> "Graph":
        """Graph over the surviving ranks after peers were lost: the lost nodes'
        edges are dropped and W is re-normalised with Metropolis weights (ranks are
        renumbered in their original order)."""
        keep = [r for r in range(self._n) if r not in set(lost)]
        if self._rank not in keep:
            raise ValueError("this rank is among the lost ones")
        adj = (self._w[np.ix_(keep, keep)] != 0).astype(float)
        w = metropolis_matrix(adj)
        return Graph(
            self.topology + "_survivors",
            len(keep),
            keep.index(self._rank),
            self._n_sub,
            None,
            self.comm_device,
            self._on_cuda,
            matrix=w,
        )

    def __repr__(self):
        return f"Graph({self.topology}, n={self._n}, rank={self._rank}, neighborhood={self.get_neighborhood()})"


def define_graph_topology(
    graph_topology: str,
    world=None,
    n_mpi_process: int = 1,
    n_sub_process: int = 1,
    comm_device: str = "cuda",
    on_cuda: bool = True,
    rank: int = 0,
    **_,
) -> Graph:
    """Factory with the reference's signature (``dl_code/pcode/utils/topology.py:599-632``)."""
    return Graph(graph_topology, n_mpi_process, rank, n_sub_process, world, comm_device, on_cuda)
