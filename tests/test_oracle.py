"""The CPU restatement against itself: the vectorised form of every function
must equal the loop form that follows the reference kernels line by line."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from oracle import epp_oracle as O
from tests.helpers import degrees_of, random_csr


@settings(max_examples=40, deadline=None)
@given(n=st.integers(1, 40), avg=st.floats(0.0, 6.0), seed=st.integers(0, 10_000), ps=st.integers(1, 7),
       empty=st.sampled_from([0.0, 0.3]))
def test_build_part_forms_agree(n, avg, seed, ps, empty):
    indptr, _ = random_csr(n, avg, seed, empty_frac=empty)
    for quirk in (False, True):
        a = O.build_part(ps, indptr, quirk)
        b = O.build_part_loops(ps, indptr, quirk)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    pp, p2n = O.build_part(ps, indptr)
    assert pp[-1] == indptr[-1]
    assert np.all(np.diff(pp) >= 1) and np.all(np.diff(pp) <= ps)
    assert np.array_equal(np.bincount(p2n, minlength=n), -(-np.diff(indptr) // ps))


def test_build_part_reference_quirk_drops_closing_pointer():
    indptr = np.array([0, 3, 5, 5], dtype=np.int32)       # last vertex has no edge
    pp, _ = O.build_part(2, indptr, reference_quirk=True)
    assert pp[-1] == 0                                      # EPPGCN.cpp:222-223
    assert O.build_part(2, indptr)[0][-1] == 5


@settings(max_examples=30, deadline=None)
@given(n=st.integers(1, 30), avg=st.floats(0.0, 5.0), seed=st.integers(0, 10_000), ps=st.integers(1, 5),
       layers=st.integers(1, 4), ratio=st.floats(0.0, 1.0))
def test_mask_forms_agree(n, avg, seed, ps, layers, ratio):
    indptr, indices = random_csr(n, avg, seed, empty_frac=0.2)
    rng = np.random.Generator(np.random.PCG64(seed + 1))
    pp, p2n = O.build_part(ps, indptr)
    for layer in range(1, layers + 1):
        src = rng.random(n) < ratio
        last = layer == layers
        outs = []
        for fn in (O.mask_forward, O.mask_forward_loops):
            ngh = np.zeros(0 if last else n, dtype=bool)
            em = np.full(len(indices), -1, dtype=np.int32)
            nd = np.zeros(n, dtype=np.int32)
            fn(p2n, pp, indices, src, ngh, em, nd, layers, layer)
            outs.append((ngh, em, nd))
        for x, y in zip(*outs):
            assert np.array_equal(x, y)
        ngh, em, nd = outs[0]
        rows = np.repeat(np.arange(n), np.diff(indptr))
        assert np.array_equal(em != -1, src[indices])
        assert np.array_equal(em[em != -1], rows[em != -1])
        assert nd.sum() == (em != -1).sum()


@settings(max_examples=40, deadline=None)
@given(e=st.integers(0, 300), seed=st.integers(0, 10_000), keep=st.floats(0.0, 1.0))
def test_compact_forms_agree(e, seed, keep):
    rng = np.random.Generator(np.random.PCG64(seed))
    mask = np.where(rng.random(e) < keep, rng.integers(0, 50, e), -1).astype(np.int32)
    col = rng.integers(0, 50, e).astype(np.int32)
    a, b = O.compact_back_edge(mask, col), O.compact_back_edge_loops(mask, col)
    assert a[2] == b[2] and np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    assert np.all(a[0][a[2]:] == 0) and np.all(a[1][a[2]:] == 0)


@settings(max_examples=60, deadline=None)
@given(n=st.integers(0, 80), seed=st.integers(0, 10_000), ps=st.integers(1, 9), hub=st.integers(0, 5000),
       slack=st.integers(0, 3))
def test_split_forms_agree(n, seed, ps, hub, slack):
    rng = np.random.Generator(np.random.PCG64(seed))
    deg = rng.integers(0, 12, n).astype(np.int32)
    deg[rng.random(n) < 0.4] = 0
    if n and hub:
        deg[rng.integers(0, n)] = hub
    num_edges = int(deg.sum()) + slack
    a, b = O.split_back_part(deg, num_edges, ps), O.split_back_part_loops(deg, num_edges, ps)
    assert a[1] == b[1] and np.array_equal(a[0], b[0])
    if a[1] + 1 <= num_edges:
        assert a[0][a[1]] == deg.sum()
        assert np.all(np.diff(a[0][:a[1] + 1]) >= 1) and np.all(np.diff(a[0][:a[1] + 1]) <= ps)


def test_split_reference_range():
    assert O.split_reference_valid(np.array([1023 * 4] * 2, dtype=np.int32), 4)
    assert not O.split_reference_valid(np.array([1024 * 4], dtype=np.int32), 4)        # > 1023 parts in a vertex
    assert not O.split_reference_valid(np.array([1000 * 4] * 3, dtype=np.int32), 4)    # > 2047 in a warp


def test_part_size_rules():
    deg = np.array([0, 3, 5, 0, 9], dtype=np.int32)
    assert O.count_nonzero(deg) == 3
    x = 0.65538 + 1.67431e-5 * 3 - 2.24342e-6 * 17 + 0.63641 * 17 / 3
    assert O.get_map_back_part_size(deg, 17) == int(np.floor(x + 0.5))
    # the rule goes negative on large graphs and is returned unclamped
    big = np.ones(2_000_000, dtype=np.int32)
    assert O.get_map_back_part_size(big, 35_000_000) < 0
    assert [O.bucket_back_part_size(v, 1) for v in (3, 4, 15, 16, 63, 64, 255, 256, 511, 512)] == \
        [4, 8, 8, 16, 16, 32, 32, 64, 64, 0]


def test_ginfo_counts_zero_degree_in_last_bucket():
    deg = np.array([0, 0, 1, 4, 5, 9, 10, 19, 20, 39, 40, 79, 80, 159, 160, 1000], dtype=np.int32)
    g = O.get_ginfo(deg, 1234)
    valid = 14
    np.testing.assert_allclose(g[:3], [valid / 1e4, 1234 / 1e4, 1234 / valid], rtol=1e-6)
    np.testing.assert_allclose(g[3:], np.array([2, 2, 2, 2, 2, 2, 4]) / valid, rtol=1e-6)


@settings(max_examples=25, deadline=None)
@given(n=st.integers(1, 25), avg=st.floats(0.0, 5.0), seed=st.integers(0, 10_000), dim=st.integers(1, 9))
def test_forward_forms_agree(n, avg, seed, dim):
    indptr, indices = random_csr(n, avg, seed, empty_frac=0.2)
    rng = np.random.Generator(np.random.PCG64(seed))
    feat = rng.standard_normal((n, dim)).astype(np.float32)
    deg = degrees_of(indptr)
    np.testing.assert_allclose(O.spmm_forward(indptr, indices, deg, feat),
                               O.spmm_forward_loops(indptr, indices, deg, feat), rtol=1e-12, atol=1e-14)


@settings(max_examples=20, deadline=None)
@given(n=st.integers(2, 25), avg=st.floats(0.5, 5.0), seed=st.integers(0, 10_000), dim=st.integers(1, 6),
       bs=st.integers(1, 5))
def test_backward_forms_agree_and_match_masked_transpose(n, avg, seed, dim, bs):
    indptr, indices = random_csr(n, avg, seed, empty_frac=0.1)
    rng = np.random.Generator(np.random.PCG64(seed))
    train = rng.random(n) < 0.4
    deg = degrees_of(indptr)
    path, _ = O.prepare_execution_path(indptr, indices, train, 2, 2, [bs, bs])
    d_out = rng.standard_normal((n, dim))
    for conv in path:
        a = O.ours_backward_aggregate(conv["id"], conv["partPointer"], conv["edgeList"], deg, d_out, conv["numParts"])
        b = O.ours_backward_aggregate_loops(conv["id"], conv["partPointer"], conv["edgeList"], deg, d_out,
                                            conv["numParts"])
        np.testing.assert_allclose(a, b, rtol=1e-12, atol=1e-14)
    # the last convolution keeps exactly the edges whose column is a training vertex
    last = path[-1]
    rows = np.repeat(np.arange(n), np.diff(indptr))
    keep = train[indices]
    want = np.zeros((n, dim))
    np.add.at(want, rows[keep], (deg[rows[keep]].astype(np.float64) * deg[indices[keep]])[:, None]
              * d_out[indices[keep]])
    got = O.ours_backward_aggregate(last["id"], last["partPointer"], last["edgeList"], deg, d_out, last["numParts"])
    np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-14)


def test_execution_path_is_exact_for_the_loss():
    """Gradient of a loss that reads only training rows, computed over the
    prepared path, equals the gradient over the whole graph (2 layers)."""
    n, dim, hid, cls = 40, 5, 4, 3
    from eppgcn_b200.graphs import csr_from_pairs
    rng = np.random.Generator(np.random.PCG64(3))
    indptr, indices = csr_from_pairs(n, rng.integers(0, n, 60), rng.integers(0, n, 60))
    train = rng.random(n) < 0.2
    deg = degrees_of(indptr).astype(np.float64)
    import scipy.sparse as sp
    A = sp.csr_matrix((np.ones(len(indices)), indices, indptr), shape=(n, n)).toarray()
    Ah = deg[:, None] * A * deg[None, :]
    X = rng.standard_normal((n, dim)); W1 = rng.standard_normal((dim, hid)); W2 = rng.standard_normal((hid, cls))
    H1 = Ah @ (X @ W1); R1 = np.maximum(H1, 0); H2 = Ah @ (R1 @ W2)
    G2 = np.zeros_like(H2); G2[train] = rng.standard_normal((int(train.sum()), cls))   # dL/dH2, train rows only
    # dense reference (the layer's backward aggregates with the same matrix, EPPGCN_kernel.cu:654-664)
    dP2 = Ah @ G2; dW2 = R1.T @ dP2; dR1 = dP2 @ W2.T; dH1 = dR1 * (H1 > 0); dP1 = Ah @ dH1; dW1 = X.T @ dP1
    path, _ = O.prepare_execution_path(indptr, indices, train, 2, 3, [2, 2])
    # The reference aggregates the backward with A rather than A^T; on a symmetric
    # graph they coincide, which is the setting the execution path is exact for.
    assert np.array_equal(A, A.T)
    p2, p1 = path[1], path[0]
    e2 = O.ours_backward_aggregate(p2["id"], p2["partPointer"], p2["edgeList"], deg, G2, p2["numParts"])
    np.testing.assert_allclose(e2, dP2, rtol=1e-12, atol=1e-13)
    e1 = O.ours_backward_aggregate(p1["id"], p1["partPointer"], p1["edgeList"], deg, dH1, p1["numParts"])
    # conv 1 only needs the rows that reach a training vertex within two hops; its
    # weight gradient is the quantity that must match
    np.testing.assert_allclose(X.T @ e1, dW1, rtol=1e-10, atol=1e-11)
    np.testing.assert_allclose(R1.T @ e2, dW2, rtol=1e-10, atol=1e-11)
