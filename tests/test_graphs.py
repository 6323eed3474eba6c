"""Seeded workload generators."""
import numpy as np
import torch

from eppgcn_b200 import graphs


def check_csr(g):
    n = g.num_nodes
    assert g.indptr.dtype == np.int32 and g.indices.dtype == np.int32
    assert g.indptr[0] == 0 and g.indptr[-1] == g.num_edges
    rows = np.repeat(np.arange(n), np.diff(g.indptr))
    key = rows.astype(np.int64) * n + g.indices
    assert np.all(np.diff(key) > 0), "columns must be sorted and distinct within a row"
    assert np.all(np.isin(np.arange(n, dtype=np.int64) * n + np.arange(n), key)), "one self loop per vertex"
    tkey = g.indices.astype(np.int64) * n + rows
    assert np.array_equal(np.sort(tkey), key), "graph must be symmetric"


def test_cora_shape_is_exact_and_deterministic():
    a = graphs.make_graph("cora", 0, cache=False)
    b = graphs.make_graph("cora", 0, cache=False)
    c = graphs.make_graph("cora", 1, cache=False)
    assert a.num_nodes == 2708 and a.num_edges == 10556 + 2708
    assert np.array_equal(a.indices, b.indices) and np.array_equal(a.indptr, b.indptr)
    assert not np.array_equal(a.indices, c.indices)
    check_csr(a)


def test_pubmed_shape():
    g = graphs.make_graph("pubmed", 0, cache=False)
    assert g.num_nodes == 19717 and g.num_edges == 2 * 88648 + 19717
    check_csr(g)
    assert int(g.num_edges / g.num_nodes) == 9


def test_rmat_shape():
    g = graphs.make_graph("rmat16", 0, cache=False)
    assert g.num_nodes == 1 << 16 and g.num_edges == 2 * 8 * (1 << 16) + (1 << 16)
    check_csr(g)
    assert np.diff(g.indptr).max() > 50 * g.num_edges / g.num_nodes, "R-MAT must be skewed"


def test_dataset_bag_layout():
    ds = graphs.load_workload("cora", 0)
    n, e = ds.num_nodes, ds.num_edges
    assert ds.x.shape == (n, 96) and torch.all(ds.x == 1)
    assert ds.row_pointers.dtype == torch.int32 and ds.column_index.dtype == torch.int32
    deg = np.diff(ds.graph.indptr)
    np.testing.assert_allclose(ds.degrees.numpy(), 1 / np.sqrt(deg), rtol=1e-6)
    assert ds.train_mask.dtype == torch.bool and 0.05 < ds.train_mask.float().mean() < 0.15
    assert len(ds.ngh_masks) == 1 and len(ds.edge_masks) == 2 and len(ds.node_degs) == 2
    assert ds.empty_mask.numel() == 0
    assert all(bool(torch.all(m == -1)) and m.numel() == e for m in ds.edge_masks)
    assert all(bool(torch.all(d == 0)) and d.numel() == n for d in ds.node_degs)
    assert torch.all(ds.y == 1) and ds.y.dtype == torch.long
    ref = graphs.load_workload("cora", 0, degree_norm="sqrt")
    np.testing.assert_allclose(ref.degrees.numpy(), np.sqrt(deg), rtol=1e-6)   # EPPGCN/dataset.py:118-119


def test_device_drawn_rmat_is_a_valid_symmetric_csr():
    """The torch generator behind the large workloads, run on the CPU at a small
    scale: sorted unique columns, exactly one self loop per vertex, symmetric,
    and the same graph for the same seed."""
    import torch
    indptr, indices = graphs.rmat_csr_device(10, 8, 0.57, 0.19, 0.19, 3, "cpu")
    again = graphs.rmat_csr_device(10, 8, 0.57, 0.19, 0.19, 3, "cpu")
    assert torch.equal(indptr, again[0]) and torch.equal(indices, again[1])
    ip, ix = indptr.numpy().astype(np.int64), indices.numpy().astype(np.int64)
    n = len(ip) - 1
    assert n == 1 << 10 and ip[0] == 0 and ip[-1] == len(ix) and indptr.dtype == torch.int32
    rows = np.repeat(np.arange(n), np.diff(ip))
    key = rows * n + ix
    assert np.all(np.diff(key) > 0)                                  # sorted within rows, no repeated pair
    assert np.array_equal(np.sort(ix * n + rows), key)               # every pair has its mirror
    assert int((rows == ix).sum()) == n                              # one self loop per vertex
    assert len(ix) > 8 * n                                           # most of the 2 * 8 * n draws survive


def test_file_csr_matches_scipy_on_random_lists():
    from hypothesis import given, settings, strategies as st
    from scipy.sparse import coo_matrix
    from eppgcn_b200 import loader

    @settings(max_examples=40, deadline=None)
    @given(st.integers(1, 60), st.integers(0, 400), st.integers(0, 10_000))
    def check(n, e, seed):
        rng = np.random.Generator(np.random.PCG64(seed))
        src, dst = rng.integers(0, n, e), rng.integers(0, n, e)
        indptr, indices = loader.csr_from_directed(n, src, dst)
        ref = coo_matrix((np.ones(e), (src, dst)), shape=(n, n)).tocsr()
        ref.sort_indices()
        assert np.array_equal(indptr, ref.indptr) and np.array_equal(indices, ref.indices)

    check()
