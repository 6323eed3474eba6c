"""The tiled planned aggregation (rows sorted into length classes) through the
C-ABI against the float64 oracle and against the group kernel.
Tolerance: |got - want| <= 2e-6 + 2e-5*|want| (the source rows are pre-scaled in
fp32 before the sum)."""
import numpy as np
import pytest
import torch

from eppgcn_b200 import capi
from oracle import epp_oracle as O
from tests.helpers import assert_close, degrees_of, random_csr, t

pytestmark = pytest.mark.gpu

GRAPHS = {
    "tiny":    dict(n=9, avg_deg=2.0, seed=1, empty_frac=0.3),
    "sparse":  dict(n=300, avg_deg=3.0, seed=2, empty_frac=0.2),
    "hubs":    dict(n=700, avg_deg=6.0, seed=3, hubs=3, hub_deg=650),
    "dense":   dict(n=128, avg_deg=40.0, seed=4),
    "loops":   dict(n=2000, avg_deg=1.0, seed=5, empty_frac=0.5),
    "chunk64": dict(n=400, avg_deg=64.0, seed=7),
}


def padded_rows(a, cuda, pad_to=4, poison=True):
    """[n, d] view of a buffer whose row stride is d rounded up to `pad_to` floats; the padding is NaN
    beyond the 16-byte piece the kernel is allowed to read."""
    n, d = a.shape
    ld = (d + pad_to - 1) // pad_to * pad_to
    full = torch.zeros(n, ld, device=cuda)
    if poison and ld > (d + 3) // 4 * 4:
        full[:, (d + 3) // 4 * 4:] = float("nan")
    full[:, :d] = t(a, cuda)
    return full[:, :d]


GRAPHS = dict(GRAPHS, wide=dict(n=300, avg_deg=30.0, seed=8, hubs=4, hub_deg=290),
              single=dict(n=64, avg_deg=1.0, seed=9))


def make_path(indptr, indices, ratio, layers, part_size, back_size, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    train = rng.random(len(indptr) - 1) < ratio
    path, _ = O.prepare_execution_path(indptr, indices, train, layers, part_size, [back_size] * layers)
    return path




def forward_case(cuda, indptr, indices, dim, pad_to=4, seed=0, out=None):
    n = len(indptr) - 1
    rng = np.random.Generator(np.random.PCG64(seed))
    feat = rng.standard_normal((n, dim)).astype(np.float32)
    deg = degrees_of(indptr)
    col = t(indices, cuda) if len(indices) else torch.zeros(0, dtype=torch.int32, device=cuda)
    plan = capi.TilePlan.from_csr(t(indptr, cuda), col)
    src = padded_rows(feat * deg[:, None], cuda, pad_to)
    got = capi.spmm_tiles(src, plan, t(deg, cuda), out=out)
    torch.cuda.synchronize()
    return got.cpu().numpy(), O.spmm_forward(indptr, indices, deg, feat), plan


@pytest.mark.parametrize("graph", sorted(GRAPHS))
@pytest.mark.parametrize("dim", [1, 3, 4, 5, 16, 22, 32, 33, 64, 96, 128, 130, 200])
def test_forward_dims(cuda, graph, dim):
    indptr, indices = random_csr(**GRAPHS[graph])
    got, want, _ = forward_case(cuda, indptr, indices, dim)
    assert np.isfinite(got).all()
    assert_close(got, want, 2e-5, 2e-6, what=f"tiled forward {graph} dim {dim}")


def test_plan_counts(cuda):
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    plan = capi.TilePlan.from_csr(t(indptr, cuda), t(indices, cuda))
    info, deg = plan.info, np.diff(indptr)
    assert info["edges"] == len(indices) and info["rows"] == n
    assert info["nonempty_rows"] == int((deg > 0).sum()) and info["atomic_rows"] == int((deg > 64).sum())
    assert info["cleared_rows"] == int((deg == 0).sum() + (deg > 64).sum())
    width = np.where(deg >= 5, (deg + 7) // 8 * 8, np.where(deg >= 3, 4, deg))
    pieces = np.where(deg > 64, (deg // 64) * 64 + np.where(deg % 64 >= 5, (deg % 64 + 7) // 8 * 8,
                                                             np.where(deg % 64 >= 3, 4, deg % 64)), width)
    assert info["slots"] >= int(pieces.sum()) and info["slots"] % 8 == 0 and info["pieces"] % 480 == 0


def test_empty_graph_and_overwrite(cuda):
    n, dim = 50, 16
    indptr = np.zeros(n + 1, dtype=np.int32)
    out = torch.full((n, dim), 7.0, device=cuda)
    plan = capi.TilePlan.from_csr(t(indptr, cuda), torch.zeros(0, dtype=torch.int32, device=cuda))
    capi.spmm_tiles(torch.ones(n, dim, device=cuda), plan, torch.ones(n, device=cuda), out=out)
    assert torch.count_nonzero(out).item() == 0, "rows without edges must come back zero"


def test_one_plan_serves_every_row_width(cuda):
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    deg = degrees_of(indptr)
    plan = capi.TilePlan.from_csr(t(indptr, cuda), t(indices, cuda))
    for dim in (3, 16, 22, 40, 64, 100, 128, 140):
        feat = np.random.Generator(np.random.PCG64(dim)).standard_normal((n, dim)).astype(np.float32)
        got = capi.spmm_tiles(padded_rows(feat * deg[:, None], cuda, 4), plan, t(deg, cuda))
        assert_close(got.cpu().numpy(), O.spmm_forward(indptr, indices, deg, feat), 2e-5, 2e-6, what=f"dim {dim}")


def test_rows_that_are_not_consecutive_are_refused(cuda):
    ids = torch.tensor([0, 0, 1, 0], dtype=torch.int32, device=cuda)
    with pytest.raises(capi.EppError) as e:
        capi.TilePlan.from_ids(ids, ids.clone(), 4, 2)
    assert e.value.status == capi.EPP_ERR_BAD_ARG


def test_result_overwrites_and_is_repeatable(cuda):
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    out = torch.full((n, 16), 7.0, device=cuda)
    a, want, _ = forward_case(cuda, indptr, indices, 16, out=out)
    assert_close(a, want, 2e-5, 2e-6, what="first call into a dirty buffer")
    b, _, _ = forward_case(cuda, indptr, indices, 16, out=out)
    assert_close(b, want, 2e-5, 2e-6, what="second call into the previous result")


@pytest.mark.parametrize("dim,left,right", [(8, 8, 0), (8, 4, 4), (22, 2, 0), (5, 3, 1), (7, 1, 0), (64, 64, 64)])
def test_result_lands_in_a_column_block(cuda, dim, left, right):
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    wide = torch.full((n, left + dim + right), 7.0, device=cuda)
    got, want, _ = forward_case(cuda, indptr, indices, dim, out=wide[:, left:left + dim])
    assert_close(got, want, 2e-5, 2e-6, what="tiled forward column block")
    full = wide.cpu().numpy()
    assert (full[:, :left] == 7.0).all() and (full[:, left + dim:] == 7.0).all()


@pytest.mark.parametrize("dim", [1, 4, 16, 22, 64, 128, 150])
@pytest.mark.parametrize("ratio", [0.0, 0.02, 0.15, 1.0])
def test_backward_over_the_compacted_path(cuda, dim, ratio):
    """Plan from the compacted row ids; rows off the path come back zero."""
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    deg = degrees_of(indptr)
    rng = np.random.Generator(np.random.PCG64(dim))
    d_out = rng.standard_normal((n, dim)).astype(np.float32)
    src = padded_rows(d_out * deg[:, None], cuda, 8)
    for conv in make_path(indptr, indices, ratio, 2, 6, 8, seed=dim + 1):
        plan = capi.TilePlan.from_ids(t(conv["id"], cuda), t(conv["edgeList"], cuda), conv["valid_len"], n)
        out = torch.full((n, dim), 5.0, device=cuda)
        capi.spmm_tiles(src, plan, t(deg, cuda), out=out)
        want = O.ours_backward_aggregate(conv["id"], conv["partPointer"], conv["edgeList"], deg, d_out,
                                         conv["numParts"])
        got = out.cpu().numpy()
        assert_close(got, want, 2e-5, 2e-6, what=f"tiled backward dim {dim} ratio {ratio}")
        assert np.all(got[conv["node_degs"] == 0] == 0), "rows off the path must come back zero"
        assert plan.info["nonempty_rows"] == int((conv["node_degs"] > 0).sum())


@pytest.mark.parametrize("dim", [16, 22, 64])
def test_agrees_with_the_group_kernel_on_rmat(cuda, dim):
    """Both kernels on a power-law graph with hub rows of tens of thousands of edges."""
    from eppgcn_b200 import graphs
    g = graphs.make_graph("rmat16", 0)
    n, e = g.num_nodes, g.num_edges
    deg = degrees_of(g.indptr)
    pp, p2n = O.build_part(max(e // n, 1), g.indptr)
    gen = torch.Generator(device=cuda).manual_seed(dim)
    ld = (dim + 7) // 8 * 8
    src = torch.randn(n, ld, device=cuda, generator=gen)[:, :dim]
    row, col, d = t(g.indptr, cuda), t(g.indices, cuda), t(deg, cuda)
    a = capi.spmm_forward(src, row, col, d, t(pp, cuda), t(p2n, cuda), e // n, prescaled=True)
    b = capi.spmm_tiles(src, capi.TilePlan.from_csr(row, col), d)
    scale = a.abs().max().item()
    assert torch.allclose(a, b, rtol=2e-5, atol=2e-6 * scale)


def test_small_cases_under_the_bounds_checking_build(cuda):
    """The library compiled with -DEPP_DEBUG_BOUNDS (the stand-in for a memory checker): clean runs
    leave its record empty, ids beyond their limit are reported and skipped.  Runs in a child process
    because the choice of library is made when ``capi`` is imported."""
    import os
    import subprocess
    import sys
    from eppgcn_b200 import build
    build.build_library(debug_bounds=True)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, EPPGCN_B200_DEBUG_BOUNDS="1", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "tests.bounds_cases"], cwd=root, env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and "bounds cases ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("dim", [1, 5, 7, 16, 22, 64])
@pytest.mark.parametrize("view", ["dense", "column_block"])
def test_pack_scaled_rows_writes_the_rows_the_path_names(cuda, dim, view):
    """The backward's source: deg[r] * d_out[r] for the rows the compacted edges name, into padded rows;
    every other row of the buffer is left alone."""
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    deg = degrees_of(indptr)
    conv = make_path(indptr, indices, 0.1, 2, 6, 8, seed=dim)[1]
    plan = capi.TilePlan.from_ids(t(conv["id"], cuda), t(conv["edgeList"], cuda), conv["valid_len"], n)
    rng = np.random.Generator(np.random.PCG64(dim))
    x = rng.standard_normal((n, dim + 3)).astype(np.float32)
    xd = t(x, cuda)
    xv = xd[:, 1:1 + dim] if view == "column_block" else xd[:, :dim].contiguous()     # 4-byte or row aligned source
    ld = (dim + 7) // 8 * 8
    dst = torch.full((n, ld), 7.0, device=cuda)
    capi.pack_scaled_rows(xv, t(deg, cuda), plan, out=dst[:, :dim])
    used = np.zeros(n, dtype=bool)
    used[conv["edgeList"][:conv["valid_len"]]] = True
    got = dst.cpu().numpy()
    want = xv.cpu().numpy() * deg[:, None]
    np.testing.assert_array_equal(got[used][:, :dim], want[used])
    assert (got[~used] == 7.0).all(), "rows no edge names must not be written"
    # and the aggregation over the packed rows equals the oracle's
    out = capi.spmm_tiles(dst[:, :dim], plan, t(deg, cuda))
    want_agg = O.ours_backward_aggregate(conv["id"], conv["partPointer"], conv["edgeList"], deg,
                                         xv.cpu().numpy(), conv["numParts"])
    assert_close(out.cpu().numpy(), want_agg, 2e-5, 2e-6, what=f"backward over packed rows dim {dim}")
    all_rows = capi.pack_scaled_rows(xv, t(deg, cuda))
    np.testing.assert_array_equal(all_rows.cpu().numpy(), want)


@pytest.mark.parametrize("dim", [1, 3, 5, 7, 21])
def test_group_kernel_writes_the_last_column_of_an_odd_row_into_an_aligned_view(cuda, dim):
    """Odd row width, source rows padded to 16 bytes, and a result view whose
    stride and base allow 8- or 16-byte stores: the last column has no partner
    in a two-float store and must still be written, forward and backward."""
    indptr, indices = random_csr(**GRAPHS["hubs"])
    n = len(indptr) - 1
    deg = degrees_of(indptr)
    rng = np.random.Generator(np.random.PCG64(dim))
    feat = rng.standard_normal((n, dim)).astype(np.float32)
    pp, p2n = O.build_part(6, indptr)
    src = padded_rows(feat, cuda, 4, poison=False)
    for stride in ((dim + 1) // 2 * 2, (dim + 3) // 4 * 4 + 4):
        wide = torch.full((n, stride), 7.0, device=cuda)
        capi.spmm_forward(src, t(indptr, cuda), t(indices, cuda), t(deg, cuda), t(pp, cuda), t(p2n, cuda), 6,
                          out=wide[:, :dim])
        assert_close(wide[:, :dim].cpu().numpy(), O.spmm_forward(indptr, indices, deg, feat),
                     what=f"forward dim {dim} stride {stride}")
        conv = make_path(indptr, indices, 0.2, 1, 6, 8, seed=dim)[0]
        wide.fill_(7.0)
        capi.spmm_backward_compacted(src, t(conv["id"], cuda), t(conv["partPointer"], cuda),
                                     t(conv["edgeList"], cuda), t(deg, cuda), conv["numParts"], 8,
                                     out=wide[:, :dim])
        want = O.ours_backward_aggregate(conv["id"], conv["partPointer"], conv["edgeList"], deg, feat,
                                         conv["numParts"])
        assert_close(wide[:, :dim].cpu().numpy(), want, what=f"backward dim {dim} stride {stride}")
        assert (wide[:, dim:].cpu().numpy() == 7.0).all()


@pytest.mark.parametrize("dim,left", [(16, 0), (22, 2), (5, 3), (64, 0)])
@pytest.mark.parametrize("graph", ["hubs", "loops"])
def test_an_edge_list_cut_into_three_plans_adds_up(cuda, graph, dim, left):
    """The edge list cut by source id into three plans over the same rows: the first stored, the others
    added (the aggregation of a row exchange that is read owner by owner)."""
    indptr, indices = random_csr(**GRAPHS[graph])
    n = len(indptr) - 1
    rng = np.random.Generator(np.random.PCG64(dim))
    feat = rng.standard_normal((n, dim)).astype(np.float32)
    deg = degrees_of(indptr)
    src = padded_rows(feat * deg[:, None], cuda)
    rows = np.repeat(np.arange(n, dtype=np.int32), np.diff(indptr))
    part = indices % 3
    wide = torch.full((n, left + dim + 1), 7.0, device=cuda)
    out = wide[:, left:left + dim]
    for k in range(3):
        pick = part == k
        plan = capi.TilePlan.from_ids(t(rows[pick], cuda), t(indices[pick].astype(np.int32), cuda), int(pick.sum()), n)
        if k == 0:
            capi.spmm_tiles(src, plan, t(deg, cuda), out=out)
        else:
            capi.spmm_tiles_add(src, plan, t(deg, cuda), out)
    torch.cuda.synchronize()
    assert_close(out.cpu().numpy(), O.spmm_forward(indptr, indices, deg, feat), 2e-5, 2e-6, what="three plans")
    full = wide.cpu().numpy()
    assert (full[:, :left] == 7.0).all() and (full[:, left + dim:] == 7.0).all()
