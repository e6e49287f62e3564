import numpy as np
import pytest

from chocosgd_b200.parallel.topology import Graph, define_graph_topology, mixing_matrix, spectral_gap


@pytest.mark.parametrize(
    "topo,n",
    [("complete", 1), ("complete", 8), ("ring", 1), ("ring", 2), ("ring", 3), ("ring", 8), ("ring", 9),
     ("torus", 9), ("torus", 12), ("torus", 16), ("margulis_expander", 9), ("margulis_expander", 16),
     ("social", 32), ("ring_ext", 8), ("expander", 7)],
)
def test_doubly_stochastic(topo, n):
    w = mixing_matrix(topo, n)
    assert w.shape == (n, n)
    np.testing.assert_allclose(w.sum(axis=1), 1.0, atol=1e-12)
    np.testing.assert_allclose(w.sum(axis=0), 1.0, atol=1e-12)
    np.testing.assert_allclose(w, w.T, atol=1e-12)
    assert (w >= -1e-12).all()


def test_ring_weights_and_neighbourhood():
    g = define_graph_topology("ring", world="0,0,0,0,0,0,0,0", n_mpi_process=8, n_sub_process=1,
                              comm_device="cuda", on_cuda=False, rank=3)
    nb = g.get_neighborhood()
    assert sorted(nb) == [2, 3, 4]
    assert all(abs(v - 1 / 3) < 1e-12 for v in nb.values())
    assert g.scaling == 3
    assert g.neighbors() == [2, 4]
    assert g.ranks == list(range(8))
    assert g.device == [0]
    # n = 2 uses the 1/2 rule of the convex code, n = 1 is the identity
    assert Graph("ring", 2, 0).get_neighborhood() == {0: 0.5, 1: 0.5}
    assert Graph("ring", 1, 0).get_neighborhood() == {0: 1.0}


def test_ring_wraparound():
    assert sorted(Graph("ring", 8, 0).get_neighborhood()) == [0, 1, 7]
    assert sorted(Graph("ring", 8, 7).get_neighborhood()) == [0, 6, 7]


def test_complete_and_spectral_gap():
    g = Graph("complete", 8, 2)
    assert len(g.get_neighborhood()) == 8 and g.scaling == 8
    assert abs(g.rho - 1.0) < 1e-9
    # ring gap 1 - (1 + 2 cos(2 pi / n)) / 3
    for n in (4, 8, 9, 16):
        expect = 1 - (1 + 2 * np.cos(2 * np.pi / n)) / 3
        assert abs(spectral_gap(mixing_matrix("ring", n)) - expect) < 1e-9


def test_torus_degree_and_shape():
    g = Graph("torus", 16, 5)
    assert len(g.get_neighborhood()) == 5
    assert all(abs(v - 0.2) < 1e-12 for v in g.get_neighborhood().values())
    # 12 nodes -> 3 x 4 grid
    w = mixing_matrix("torus", 12)
    assert ((w > 0).sum(axis=1) == 5).all()


def test_torus_matches_networkx():
    networkx = pytest.importorskip("networkx")
    for n in (9, 12, 16):
        m = int(np.sqrt(n))
        while n % m:
            m -= 1
        g = networkx.generators.lattice.grid_2d_graph(m, n // m, periodic=True)
        a = networkx.to_numpy_array(g)
        np.fill_diagonal(a, 1)
        np.testing.assert_allclose(mixing_matrix("torus", n), a / 5)


def test_margulis_matches_networkx():
    networkx = pytest.importorskip("networkx")
    g = networkx.generators.expanders.margulis_gabber_galil_graph(4)
    a = networkx.to_numpy_array(g)
    a[a > 1] = 1
    from chocosgd_b200.parallel.topology import max_degree_weights

    np.testing.assert_allclose(mixing_matrix("margulis_expander", 16), max_degree_weights(a), atol=1e-12)


def test_survivor_graph():
    g = Graph("ring", 8, 3).without([4])
    assert g.n_nodes == 7
    w = g.matrix
    np.testing.assert_allclose(w.sum(axis=1), 1.0)
    np.testing.assert_allclose(w, w.T)
    assert g.rank == 3


def test_world_mapping():
    g = Graph("ring", 4, 1, n_sub_process=2, world="0,1,2,3,4,5,6,7")
    assert g.device == [2, 3]
    with pytest.raises(ValueError):
        Graph("ring", 4, 1, n_sub_process=2, world="0,1")
