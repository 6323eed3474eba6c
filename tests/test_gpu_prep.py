"""Execution-path preparation kernels through the C-ABI: bit-exact against the
oracle, in both scan modes, and identical when repeated."""
import numpy as np
import pytest
import torch

from eppgcn_b200 import capi
from oracle import epp_oracle as O
from tests.helpers import random_csr, t

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("layers", [1, 2, 3, 4])
@pytest.mark.parametrize("part_size", [1, 3, 32])
def test_mask_forward_chain(cuda, layers, part_size):
    indptr, indices = random_csr(n=900, avg_deg=5.0, seed=layers, empty_frac=0.15, hubs=2, hub_deg=700)
    n, e = len(indptr) - 1, len(indices)
    rng = np.random.Generator(np.random.PCG64(part_size))
    train = rng.random(n) < 0.05
    pp, p2n = O.build_part(part_size, indptr)
    d_pp, d_p2n, d_col = t(pp, cuda), t(p2n, cuda), t(indices, cuda)
    src_np, src_t = train, t(train, cuda)
    for layer in range(1, layers + 1):
        last = layer == layers
        ngh_np = np.zeros(0 if last else n, dtype=bool)
        em_np = np.full(e, -1, dtype=np.int32)
        nd_np = np.zeros(n, dtype=np.int32)
        O.mask_forward(p2n, pp, indices, src_np, ngh_np, em_np, nd_np, layers, layer)
        ngh_t = torch.zeros(0 if last else n, dtype=torch.bool, device=cuda)
        em_t = torch.full((e,), -1, dtype=torch.int32, device=cuda)
        nd_t = torch.zeros(n, dtype=torch.int32, device=cuda)
        capi.mask_forward(d_p2n, d_pp, d_col, src_t, ngh_t, em_t, nd_t, layers, layer)
        assert np.array_equal(em_t.cpu().numpy(), em_np)
        assert np.array_equal(nd_t.cpu().numpy(), nd_np)
        assert np.array_equal(ngh_t.cpu().numpy(), ngh_np)
        src_np, src_t = ngh_np, ngh_t


def test_mask_forward_accumulates_like_the_reference(cuda):
    """node_degs is added to and back_edge_mask only written where active
    (EPPGCN_kernel.cu:379-386): prior contents survive."""
    indptr, indices = random_csr(n=200, avg_deg=4.0, seed=5)
    n, e = len(indptr) - 1, len(indices)
    pp, p2n = O.build_part(4, indptr)
    src = np.random.Generator(np.random.PCG64(1)).random(n) < 0.3
    em_np = np.full(e, -7, dtype=np.int32); nd_np = np.full(n, 3, dtype=np.int32); ngh_np = np.zeros(n, dtype=bool)
    ngh_np[:10] = True
    em_t, nd_t, ngh_t = t(em_np, cuda), t(nd_np, cuda), t(ngh_np, cuda)
    O.mask_forward(p2n, pp, indices, src, ngh_np, em_np, nd_np, 2, 1)
    capi.mask_forward(t(p2n, cuda), t(pp, cuda), t(indices, cuda), t(src, cuda), ngh_t, em_t, nd_t, 2, 1)
    assert np.array_equal(em_t.cpu().numpy(), em_np) and np.array_equal(nd_t.cpu().numpy(), nd_np)
    assert np.array_equal(ngh_t.cpu().numpy(), ngh_np)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("length,keep", [(0, 0.5), (1, 1.0), (1, 0.0), (31, 0.5), (4095, 0.3), (4096, 0.3),
                                         (4097, 0.3), (50_000, 0.0), (50_000, 1.0), (1_000_003, 0.1),
                                         (1_000_003, 0.8)])
def test_compact_mask(cuda, mode, length, keep):
    rng = np.random.Generator(np.random.PCG64(length + int(keep * 10)))
    mask = np.where(rng.random(length) < keep, rng.integers(0, 1 << 20, length), -1).astype(np.int32)
    col = rng.integers(0, 1 << 20, length).astype(np.int32)
    want = O.compact_back_edge(mask, col)
    for _ in range(2):                                   # twice: the scan must be repeatable
        ids, edges, valid = capi.compact_mask(t(mask, cuda), t(col, cuda), mode)
        assert valid == want[2]
        assert np.array_equal(ids.cpu().numpy(), want[0])
        assert np.array_equal(edges.cpu().numpy(), want[1])


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("n,part_size,hub", [(1, 1, 0), (5, 3, 0), (2047, 4, 0), (2048, 4, 0), (2049, 4, 0),
                                            (100_000, 1, 0), (100_000, 32, 0), (70_000, 2, 300_000),
                                            (70_000, 64, 2_000_000), (5000, 1_000_000, 50)])
def test_split_parts(cuda, mode, n, part_size, hub):
    rng = np.random.Generator(np.random.PCG64(n + part_size))
    deg = rng.integers(0, 40, n).astype(np.int32)
    deg[rng.random(n) < 0.5] = 0
    if hub:
        deg[rng.integers(0, n, 3)] = hub                  # far beyond the reference's 1023 parts per vertex
    num_edges = int(deg.astype(np.int64).sum()) + 5
    want, want_parts = O.split_back_part(deg, num_edges, part_size, out_len=num_edges + 1)
    for _ in range(2):
        pp, parts = capi.split_parts(t(deg, cuda), num_edges, part_size, mode)
        assert parts == want_parts
        assert np.array_equal(pp.cpu().numpy(), want)


def test_split_drops_the_entry_that_does_not_fit(cuda):
    deg = np.array([2, 0, 3], dtype=np.int32)             # five single-edge parts, closing pointer is the sixth
    pp, parts = capi.split_parts(t(deg, cuda), 5, 1, out_len=5)
    want, want_parts = O.split_back_part(deg, 5, 1)
    assert parts == want_parts == 5 and np.array_equal(pp.cpu().numpy(), want)


def test_split_rejects_non_positive_part_size(cuda):
    with pytest.raises(capi.EppError):
        capi.split_parts(torch.ones(4, dtype=torch.int32, device=cuda), 4, 0)


@pytest.mark.parametrize("n", [0, 1, 255, 100_001])
def test_count_nonzero(cuda, n):
    v = np.random.Generator(np.random.PCG64(n)).integers(-1, 3, n).astype(np.int32)
    assert capi.count_nonzero(t(v, cuda)) == int(np.count_nonzero(v))


def test_prepared_path_feeds_backward(cuda):
    """mask -> compact -> split on the GPU, end to end, equals the oracle."""
    indptr, indices = random_csr(n=3000, avg_deg=8.0, seed=21, hubs=2, hub_deg=2500)
    n, e = len(indptr) - 1, len(indices)
    train = np.random.Generator(np.random.PCG64(4)).random(n) < 0.1
    layers, ps, bs = 3, 8, 16
    want, _ = O.prepare_execution_path(indptr, indices, train, layers, ps, [bs] * layers)
    pp, p2n = O.build_part(ps, indptr)
    d_pp, d_p2n, d_col = t(pp, cuda), t(p2n, cuda), t(indices, cuda)
    ngh = [torch.zeros(n, dtype=torch.bool, device=cuda) for _ in range(layers - 1)]
    ems = [torch.full((e,), -1, dtype=torch.int32, device=cuda) for _ in range(layers)]
    nds = [torch.zeros(n, dtype=torch.int32, device=cuda) for _ in range(layers)]
    empty = torch.zeros(0, dtype=torch.bool, device=cuda)
    for i in range(layers):
        src = t(train, cuda) if i == 0 else ngh[i - 1]
        dst = ngh[i] if i < layers - 1 else empty
        capi.mask_forward(d_p2n, d_pp, d_col, src, dst, ems[layers - 1 - i], nds[layers - 1 - i], layers, i + 1)
    for i in range(layers):
        ids, edges, valid = capi.compact_mask(ems[i], d_col)
        part_ptr, parts = capi.split_parts(nds[i], e, bs)
        w = want[i]
        assert valid == w["valid_len"] and parts == w["numParts"]
        assert np.array_equal(ids.cpu().numpy(), w["id"]) and np.array_equal(edges.cpu().numpy(), w["edgeList"])
        assert np.array_equal(part_ptr.cpu().numpy(), w["partPointer"])


def test_bounded_wait_reports_a_timeout_and_leaves_the_context_usable(cuda):
    """The look-back wait of the compaction is bounded.  Mode 2 withholds the
    first tile, so the wait of the second one must run out: the call comes back
    with EPP_ERR_SCAN_TIMEOUT instead of hanging, and the next call works."""
    import time
    rng = np.random.Generator(np.random.PCG64(1))
    mask = np.where(rng.random(100_000) < 0.5, rng.integers(0, 1000, 100_000), -1).astype(np.int32)
    col = rng.integers(0, 1000, 100_000).astype(np.int32)
    t0 = time.perf_counter()
    with pytest.raises(capi.EppError) as e:
        capi.compact_mask(t(mask, cuda), t(col, cuda), mode=2)
    assert e.value.status == capi.EPP_ERR_SCAN_TIMEOUT
    assert time.perf_counter() - t0 < 30.0
    want = O.compact_back_edge(mask, col)                      # the fallback the operator module takes
    for mode in (1, 0):
        ids, edges, valid = capi.compact_mask(t(mask, cuda), t(col, cuda), mode)
        assert valid == want[2] and np.array_equal(ids.cpu().numpy(), want[0])


@pytest.mark.parametrize("part_size", [1, 3, 17, 64, 100_000])
@pytest.mark.parametrize("mode", [0, 1])
def test_groups_built_on_the_device_equal_the_host_partition(cuda, part_size, mode):
    """eppgcn_build_part against eppgcn_build_part_host and the oracle: empty rows, an empty last
    vertex, hub rows of thousands of groups, more than one scan tile."""
    import eppgcn_b200
    rng = np.random.Generator(np.random.PCG64(part_size))
    deg = rng.poisson(3.0, 70_001)
    deg[rng.random(deg.size) < 0.3] = 0
    deg[[5, 40_000, 69_999]] = [30_000, 77_777, 12_345]
    deg[-1] = 0
    indptr = np.zeros(deg.size + 1, dtype=np.int32)
    np.cumsum(deg, out=indptr[1:])
    want_pp, want_p2n = O.build_part(part_size, indptr)
    host_pp, host_p2n = capi.build_part(part_size, torch.from_numpy(indptr))
    assert np.array_equal(host_pp.numpy(), want_pp) and np.array_equal(host_p2n.numpy(), want_p2n)
    pp, p2n = capi.build_part_device(part_size, torch.from_numpy(indptr).to(cuda), mode=mode)
    assert np.array_equal(pp.cpu().numpy(), want_pp) and np.array_equal(p2n.cpu().numpy(), want_p2n)
    if mode == 0:                                   # the operator accepts a CUDA row pointer as well
        gnna = eppgcn_b200.load_gnnadvisor()
        a, b = gnna.build_part(part_size, torch.from_numpy(indptr).to(cuda))
        assert a.is_cuda and torch.equal(a, pp) and torch.equal(b, p2n)


def test_groups_of_an_empty_graph_on_the_device(cuda):
    pp, p2n = capi.build_part_device(4, torch.zeros(11, dtype=torch.int32, device=cuda))
    assert pp.tolist() == [0] and p2n.numel() == 0
