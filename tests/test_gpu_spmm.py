"""CUDA aggregations through the C-ABI against the float64 oracle.
Tolerance: |got - want| <= 1e-6 + 1e-5*|want| (atomics reorder the sums)."""
import numpy as np
import pytest
import torch

from eppgcn_b200 import capi
from oracle import epp_oracle as O
from tests.helpers import assert_close, degrees_of, random_csr, t

pytestmark = pytest.mark.gpu

GRAPHS = {
    "tiny":   dict(n=9, avg_deg=2.0, seed=1, empty_frac=0.3),
    "sparse": dict(n=300, avg_deg=3.0, seed=2, empty_frac=0.2),
    "hubs":   dict(n=700, avg_deg=6.0, seed=3, hubs=3, hub_deg=650),
    "dense":  dict(n=128, avg_deg=40.0, seed=4),
}


def run_forward(cuda, indptr, indices, dim, part_size, pad=0, seed=0, deg_kind="rsqrt"):
    n = len(indptr) - 1
    rng = np.random.Generator(np.random.PCG64(seed))
    feat = rng.standard_normal((n, dim)).astype(np.float32)
    deg = degrees_of(indptr, deg_kind)
    pp, p2n = O.build_part(part_size, indptr)
    full = torch.full((n, dim + pad), float("nan"), device=cuda)     # padding must never leak into the result
    full[:, :dim] = t(feat, cuda)
    out = capi.spmm_forward(full[:, :dim], t(indptr, cuda), t(indices, cuda), t(deg, cuda), t(pp, cuda),
                            t(p2n, cuda), part_size)
    torch.cuda.synchronize()
    return out.cpu().numpy(), O.spmm_forward(indptr, indices, deg, feat)


@pytest.mark.parametrize("graph", sorted(GRAPHS))
@pytest.mark.parametrize("dim", [1, 2, 3, 4, 5, 8, 16, 22, 32, 33, 64, 96, 128, 130, 200])
def test_forward_dims(cuda, graph, dim):
    indptr, indices = random_csr(**GRAPHS[graph])
    got, want = run_forward(cuda, indptr, indices, dim, part_size=4)
    assert_close(got, want, what=f"forward {graph} dim {dim}")


@pytest.mark.parametrize("part_size", [1, 2, 7, 17, 32, 1000])
@pytest.mark.parametrize("dim", [16, 22, 128])
def test_forward_group_sizes(cuda, part_size, dim):
    indptr, indices = random_csr(**GRAPHS["hubs"])
    got, want = run_forward(cuda, indptr, indices, dim, part_size)
    assert_close(got, want, what=f"forward part_size {part_size} dim {dim}")


@pytest.mark.parametrize("dim,pad", [(22, 2), (22, 10), (16, 8), (5, 3), (7, 1), (3, 1), (130, 6)])
def test_forward_padded_row_stride(cuda, dim, pad):
    indptr, indices = random_csr(**GRAPHS["sparse"])
    got, want = run_forward(cuda, indptr, indices, dim, 5, pad=pad)
    assert np.isfinite(got).all()
    assert_close(got, want, what=f"forward dim {dim} stride {dim + pad}")


def test_forward_reference_degree_convention(cuda):
    """The operator multiplies whatever `degrees` holds; the reference loader
    stores sqrt(deg) (EPPGCN/dataset.py:118-119)."""
    indptr, indices = random_csr(**GRAPHS["sparse"])
    got, want = run_forward(cuda, indptr, indices, 16, 3, deg_kind="sqrt")
    assert_close(got, want, what="sqrt degrees")


def test_forward_empty_graph_and_overwrite(cuda):
    n, dim = 50, 16
    indptr = np.zeros(n + 1, dtype=np.int32)
    out = torch.full((n, dim), 7.0, device=cuda)
    z = torch.zeros(0, dtype=torch.int32, device=cuda)
    capi.spmm_forward(torch.ones(n, dim, device=cuda), t(indptr, cuda), z, torch.ones(n, device=cuda),
                      torch.zeros(1, dtype=torch.int32, device=cuda), z, 4, out=out)
    assert torch.count_nonzero(out).item() == 0, "rows without edges must come back zero"


def test_forward_is_linear_and_repeatable(cuda):
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    deg = degrees_of(indptr)
    pp, p2n = O.build_part(8, indptr)
    args = [t(a, cuda) for a in (indptr, indices, deg, pp, p2n)]
    g = torch.Generator(device=cuda).manual_seed(1)
    a = torch.randn(n, 32, device=cuda, generator=g)
    b = torch.randn(n, 32, device=cuda, generator=g)
    fa, fb, fab = (capi.spmm_forward(x, *args, 8) for x in (a, b, 2 * a - 3 * b))
    torch.testing.assert_close(fab, 2 * fa - 3 * fb, rtol=1e-4, atol=1e-5)
    again = capi.spmm_forward(a, *args, 8)
    torch.testing.assert_close(again, fa, rtol=1e-5, atol=1e-6)


def make_path(indptr, indices, ratio, layers, part_size, back_size, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    train = rng.random(len(indptr) - 1) < ratio
    path, _ = O.prepare_execution_path(indptr, indices, train, layers, part_size, [back_size] * layers)
    return path


@pytest.mark.parametrize("dim", [1, 3, 4, 16, 22, 32, 64, 128, 150])
@pytest.mark.parametrize("back_size", [1, 4, 32])
def test_backward_compacted(cuda, dim, back_size):
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    deg = degrees_of(indptr)
    rng = np.random.Generator(np.random.PCG64(dim))
    d_out = rng.standard_normal((n, dim)).astype(np.float32)
    for conv in make_path(indptr, indices, 0.15, 2, 6, back_size, seed=dim):
        got = capi.spmm_backward_compacted(t(d_out, cuda), t(conv["id"], cuda), t(conv["partPointer"], cuda),
                                           t(conv["edgeList"], cuda), t(deg, cuda), conv["numParts"], back_size)
        want = O.ours_backward_aggregate(conv["id"], conv["partPointer"], conv["edgeList"], deg, d_out,
                                         conv["numParts"])
        assert_close(got.cpu().numpy(), want, what=f"backward dim {dim} size {back_size}")


@pytest.mark.parametrize("ratio", [0.0, 0.01, 0.5, 1.0])
def test_backward_train_ratios(cuda, ratio):
    indptr, indices = random_csr(**GRAPHS["sparse"])
    n = len(indptr) - 1
    deg = degrees_of(indptr)
    d_out = np.random.Generator(np.random.PCG64(9)).standard_normal((n, 16)).astype(np.float32)
    for conv in make_path(indptr, indices, ratio, 3, 4, 8, seed=11):
        out = torch.full((n, 16), 5.0, device=cuda)
        capi.spmm_backward_compacted(t(d_out, cuda), t(conv["id"], cuda), t(conv["partPointer"], cuda),
                                     t(conv["edgeList"], cuda), t(deg, cuda), conv["numParts"], 8, out=out)
        want = O.ours_backward_aggregate(conv["id"], conv["partPointer"], conv["edgeList"], deg, d_out,
                                         conv["numParts"])
        assert_close(out.cpu().numpy(), want, what=f"backward ratio {ratio}")
        off_path = conv["node_degs"] == 0
        assert np.all(out.cpu().numpy()[off_path] == 0), "rows off the path must come back zero"


@pytest.mark.parametrize("n,k,dout", [(1, 1, 1), (127, 3, 4), (128, 12, 16), (129, 96, 16), (1000, 128, 22),
                                      (333, 130, 32), (2049, 16, 22), (64, 7, 5)])
@pytest.mark.parametrize("scaled", [True, False])
def test_update_scaled(cuda, n, k, dout, scaled):
    """diag(scale) (X W) with FP32 FMA against float64; K-long fp32 dot products."""
    rng = np.random.Generator(np.random.PCG64(n + k + dout))
    kp = (k + 3) // 4 * 4
    x_full = torch.full((n, kp), float("nan"), device=cuda)                  # row stride padded to 16 bytes
    x = rng.standard_normal((n, k)).astype(np.float32)
    x_full[:, :k] = t(x, cuda)
    w = rng.uniform(-0.5, 0.5, (k, dout)).astype(np.float32)
    s = rng.uniform(0.1, 2.0, n).astype(np.float32)
    got = capi.update_scaled(x_full[:, :k], t(w, cuda), t(s, cuda) if scaled else None)
    assert got.shape == (n, dout) and got.stride(0) % 8 == 0
    want = x.astype(np.float64) @ w.astype(np.float64)
    if scaled:
        want *= s.astype(np.float64)[:, None]
    mag = np.abs(x.astype(np.float64)) @ np.abs(w.astype(np.float64)) * (s[:, None] if scaled else 1.0)
    err = np.abs(got.cpu().numpy() - want)
    assert np.all(err <= 1e-6 + 4e-7 * mag * max(1, int(np.sqrt(k)))), f"worst {err.max():.3e}"
    pad = got.stride(0) - dout
    if pad:                                                                   # padding columns are zeroed
        full = torch.as_strided(got, (n, got.stride(0)), (got.stride(0), 1))
        assert torch.count_nonzero(full[:, dout:]).item() == 0


def test_update_rejects_wide_outputs(cuda):
    with pytest.raises(capi.EppError) as e:
        capi.update_scaled(torch.zeros(8, 8, device=cuda), torch.zeros(8, 33, device=cuda))
    assert e.value.status == capi.EPP_ERR_TOO_LARGE


@pytest.mark.parametrize("dim", [1, 16, 22, 64, 128])
def test_forward_prescaled_rows(cuda, dim):
    """deg_col = NULL: rows that already carry deg[col] give the same result."""
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    deg = degrees_of(indptr)
    feat = np.random.Generator(np.random.PCG64(dim)).standard_normal((n, dim)).astype(np.float32)
    pp, p2n = O.build_part(6, indptr)
    scaled = t(feat * deg[:, None], cuda)
    got = capi.spmm_forward(scaled, t(indptr, cuda), t(indices, cuda), t(deg, cuda), t(pp, cuda), t(p2n, cuda), 6,
                            prescaled=True)
    assert_close(got.cpu().numpy(), O.spmm_forward(indptr, indices, deg, feat), 2e-5, 2e-6, f"prescaled dim {dim}")


@pytest.mark.parametrize("n,k,dout", [(1, 4, 4), (31, 16, 22), (32, 16, 22), (1000, 128, 16), (5000, 7, 5),
                                      (100_003, 128, 16), (4097, 128, 32), (70_000, 16, 22), (3000, 200, 20),
                                      (2000, 1000, 4), (999, 22, 16), (777, 40, 28), (50_000, 64, 32), (9, 3, 1)])
def test_weight_grad(cuda, n, k, dout):
    """X^T d' with FP32 FMA and atomically combined slabs, against float64."""
    rng = np.random.Generator(np.random.PCG64(n + k))
    x = rng.standard_normal((n, k)).astype(np.float32)
    d = rng.standard_normal((n, dout)).astype(np.float32)
    d[rng.random(n) < 0.5] = 0.0                                   # rows off the execution path
    got = capi.weight_grad(t(x, cuda), t(d, cuda)).cpu().numpy()
    want = x.astype(np.float64).T @ d.astype(np.float64)
    mag = np.abs(x.astype(np.float64)).T @ np.abs(d.astype(np.float64))
    assert got.shape == (k, dout)
    assert np.all(np.abs(got - want) <= 1e-6 + 1e-6 * mag * max(1.0, np.sqrt(n) / 8)), \
        f"worst {np.abs(got - want).max():.3e}"


def test_weight_grad_limits(cuda):
    with pytest.raises(capi.EppError) as e:
        capi.weight_grad(torch.zeros(8, 512, device=cuda), torch.zeros(8, 32, device=cuda))
    assert e.value.status == capi.EPP_ERR_TOO_LARGE


def test_operator_backward_products_match_float64(cuda):
    """ours_backward's d_input and d_weight through the FMA kernels (Din 128 -> four 32-column launches)."""
    import eppgcn_b200
    gnna = eppgcn_b200.load_gnnadvisor()
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    deg = degrees_of(indptr)
    rng = np.random.Generator(np.random.PCG64(3))
    for din, dout in ((128, 16), (16, 22)):
        x = rng.standard_normal((n, din)).astype(np.float32)
        w = rng.uniform(-0.3, 0.3, (din, dout)).astype(np.float32)
        d_out = rng.standard_normal((n, dout)).astype(np.float32)
        conv = make_path(indptr, indices, 0.2, 1, 6, 8, seed=din)[0]
        d_in, d_w = gnna.ours_backward(t(d_out, cuda), t(x, cuda), t(w, cuda), t(conv["id"], cuda),
                                       t(conv["partPointer"], cuda), t(conv["edgeList"], cuda), t(deg, cuda),
                                       8, conv["numParts"], 1, 4, 16)
        wi, ww, _ = O.gcn_layer_backward(d_out, x, w, conv["id"], conv["partPointer"], conv["edgeList"], deg,
                                         conv["numParts"])
        assert d_in.shape == (n, din) and d_w.shape == (din, dout)
        assert_close(d_in.cpu().numpy(), wi, 2e-5, 2e-6, f"d_input {din}->{dout}")
        s = float(np.abs(ww).max())
        assert_close(d_w.cpu().numpy() / s, ww / s, 1e-4, 1e-5, f"d_weight {din}->{dout}")


@pytest.mark.parametrize("dim,left,right", [(8, 8, 0), (8, 4, 4), (22, 2, 0), (5, 3, 1), (64, 64, 64)])
def test_results_land_in_a_column_block_of_a_wider_matrix(cuda, dim, left, right):
    """Output rows with a stride: forward and compacted backward fill columns
    left .. left+dim of a wider matrix and leave the columns on either side alone."""
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    rng = np.random.Generator(np.random.PCG64(5))
    feat = rng.standard_normal((n, dim)).astype(np.float32)
    deg = degrees_of(indptr, "rsqrt")
    pp, p2n = O.build_part(6, indptr)
    wide = torch.full((n, left + dim + right), 7.0, device=cuda)
    capi.spmm_forward(t(feat, cuda), t(indptr, cuda), t(indices, cuda), t(deg, cuda), t(pp, cuda), t(p2n, cuda), 6,
                      out=wide[:, left:left + dim])
    got = wide.cpu().numpy()
    assert_close(got[:, left:left + dim], O.spmm_forward(indptr, indices, deg, feat), what="forward column block")
    assert (got[:, :left] == 7.0).all() and (got[:, left + dim:] == 7.0).all()

    train = rng.random(n) < 0.2
    path, _ = O.prepare_execution_path(indptr, indices, train, 1, 6, [8])
    conv = path[0]
    wide.fill_(7.0)
    capi.spmm_backward_compacted(t(feat, cuda), t(conv["id"], cuda), t(conv["partPointer"], cuda),
                                 t(conv["edgeList"], cuda), t(deg, cuda), conv["numParts"], 8,
                                 out=wide[:, left:left + dim])
    got = wide.cpu().numpy()
    want = O.ours_backward_aggregate(conv["id"], conv["partPointer"], conv["edgeList"], deg, feat, conv["numParts"])
    assert_close(got[:, left:left + dim], want, what="backward column block")
    assert (got[:, :left] == 7.0).all() and (got[:, left + dim:] == 7.0).all()


def test_weight_grad_over_the_rows_of_a_path(cuda):
    """X^T d' restricted to the rows that have edges in a plan: d' is zero everywhere else, so the
    product equals the one over all rows."""
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    conv = make_path(indptr, indices, 0.05, 2, 6, 8, seed=4)[1]
    plan = capi.TilePlan.from_ids(t(conv["id"], cuda), t(conv["edgeList"], cuda), conv["valid_len"], n)
    active = conv["node_degs"] > 0
    assert 0 < active.sum() < n
    rng = np.random.Generator(np.random.PCG64(8))
    for k, dout in ((128, 16), (16, 22), (12, 5)):
        x = rng.standard_normal((n, k)).astype(np.float32)
        d = rng.standard_normal((n, dout)).astype(np.float32)
        d[~active] = 0.0
        got = capi.weight_grad(t(x, cuda), t(d, cuda), plan).cpu().numpy()
        want = x.astype(np.float64).T @ d.astype(np.float64)
        mag = np.abs(x.astype(np.float64)).T @ np.abs(d.astype(np.float64))
        assert np.all(np.abs(got - want) <= 1e-6 + 1e-6 * mag * max(1.0, np.sqrt(n) / 8)), f"k {k} dout {dout}"
        # rows off the list are not read at all: poison them
        x[~active] = np.nan
        got = capi.weight_grad(t(x, cuda), t(d, cuda), plan).cpu().numpy()
        assert np.isfinite(got).all()


@pytest.mark.parametrize("din,dout", [(128, 64), (64, 64), (64, 32), (40, 36)])
def test_operator_handles_wide_layers_without_library_gemms(cuda, din, dout):
    """forward and ours_backward for layers wider than one 32-column block (the 3-layer configuration:
    128 -> 64 -> 64 -> 32): update, d_input and d_weight go through this library's FMA kernels block
    by block and match float64."""
    import eppgcn_b200
    gnna = eppgcn_b200.load_gnnadvisor()
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    deg = degrees_of(indptr)
    rng = np.random.Generator(np.random.PCG64(din + dout))
    x = rng.standard_normal((n, din)).astype(np.float32)
    w = rng.uniform(-0.3, 0.3, (din, dout)).astype(np.float32)
    pp, p2n = O.build_part(6, indptr)
    y = gnna.forward(t(x, cuda), t(w, cuda), t(indptr, cuda), t(indices, cuda), t(deg, cuda), t(pp, cuda),
                     t(p2n, cuda), 6, 32, 8)[0]
    assert_close(y.cpu().numpy(), O.gcn_layer_forward(x, w, indptr, indices, deg), 4e-5, 4e-6, f"forward {din}->{dout}")
    d_out = rng.standard_normal((n, dout)).astype(np.float32)
    conv = make_path(indptr, indices, 0.2, 1, 6, 8, seed=din)[0]
    args = (t(d_out, cuda), t(x, cuda), t(w, cuda), t(conv["id"], cuda), t(conv["partPointer"], cuda),
            t(conv["edgeList"], cuda), t(deg, cuda), 8, conv["numParts"], 1, 4, 16)
    d_in, d_w = gnna.ours_backward(*args)
    wi, ww, _ = O.gcn_layer_backward(d_out, x, w, conv["id"], conv["partPointer"], conv["edgeList"], deg,
                                     conv["numParts"])
    assert_close(d_in.cpu().numpy(), wi, 4e-5, 4e-6, f"d_input {din}->{dout}")
    s = float(np.abs(ww).max())
    assert_close(d_w.cpu().numpy() / s, ww / s, 1e-4, 1e-5, f"d_weight {din}->{dout}")
    none, d_w2 = gnna.ours_backward_weight_only(*args)
    assert none.numel() == 0
    assert_close(d_w2.cpu().numpy() / s, ww / s, 1e-4, 1e-5, f"d_weight (weight only) {din}->{dout}")
