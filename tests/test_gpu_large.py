"""Parity at the sizes that are benchmarked: the 2-million-vertex R-MAT graph
and the 1.13-million-vertex social-shaped graph at train ratios 0.01 / 0.1 /
0.5.  Preparation (mask -> compaction -> splitting) is compared bit for bit
with the vectorised numpy oracle on the full arrays; the forward and the
compacted backward aggregation of both kernels (group kernel, tiled planned kernel)
are compared with the float64 oracle on every row.
Tolerance: |got - want| <= 1e-6 + 1e-5*|want|; twice that where the source rows
were scaled in fp32 before the sum (pre-scaled rows)."""
import numpy as np
import pytest
import torch

import eppgcn_b200
from eppgcn_b200 import capi, graphs
from oracle import epp_oracle as O
from tests.helpers import assert_close, t

pytestmark = pytest.mark.gpu

CASES = [("rmat21", 0.1), ("social", 0.01), ("social", 0.1), ("social", 0.5)]
BACK = 32


@pytest.fixture(scope="module", params=CASES, ids=[f"{w}-r{r}" for w, r in CASES])
def prepared(request, cuda):
    """Device-side preparation through the operator module beside the oracle's."""
    workload, ratio = request.param
    gnna = eppgcn_b200.load_gnnadvisor()
    ds = graphs.load_workload(workload, 0, train_ratio=ratio)
    ip, ix = ds.graph.indptr, ds.graph.indices
    n, e, L = ds.num_nodes, ds.num_edges, 2
    part = max(int(ds.avg_degree), 1)
    train = ds.train_mask.numpy().copy()
    deg = ds.degrees.numpy().copy()
    pp, p2n = gnna.build_part(part, ds.row_pointers)
    want_pp, want_p2n = O.build_part(part, ip)
    assert np.array_equal(pp.numpy(), want_pp) and np.array_equal(p2n.numpy(), want_p2n)
    row, col = ds.row_pointers.to(cuda), ds.column_index.to(cuda)
    pp, p2n = pp.to(cuda), p2n.to(cuda)
    ds.to(cuda)
    for i in range(L):
        src = ds.train_mask if i == 0 else ds.ngh_masks[i - 1]
        dst = ds.ngh_masks[i] if i < L - 1 else ds.empty_mask
        gnna.mask_forward(p2n, pp, col, src, dst, ds.edge_masks[L - 1 - i], ds.node_degs[L - 1 - i], L, i + 1, 4, 16)
    path = []
    for i in range(L):
        ids, edges, info = gnna.compact_back_edge(ds.edge_masks[i], col)
        ppb, pinfo = gnna.split_back_part(ds.node_degs[i], e, BACK)
        path.append(dict(id=ids, edges=edges, pp=ppb, parts=int(pinfo[0].item()), valid=int(info[0].item())))
    want, want_ngh = O.prepare_execution_path(ip, ix, train, L, part, [BACK] * L)
    return dict(ds=ds, n=n, e=e, ip=ip, ix=ix, deg=deg, part=part, row=row, col=col, pp=pp, p2n=p2n,
                degd=ds.degrees, path=path, want=want, want_ngh=want_ngh, workload=workload, ratio=ratio)


def test_preparation_is_bit_exact_on_the_full_arrays(prepared):
    P = prepared
    ds = P["ds"]
    assert np.array_equal(ds.ngh_masks[0].cpu().numpy(), P["want_ngh"][0])
    for i, (got, want) in enumerate(zip(P["path"], P["want"])):
        assert np.array_equal(ds.edge_masks[i].cpu().numpy(), want["edge_mask"]), f"edge mask of conv {i + 1}"
        assert np.array_equal(ds.node_degs[i].cpu().numpy(), want["node_degs"]), f"node degrees of conv {i + 1}"
        assert got["valid"] == want["valid_len"] and got["parts"] == want["numParts"]
        assert np.array_equal(got["id"].cpu().numpy(), want["id"])
        assert np.array_equal(got["edges"].cpu().numpy(), want["edgeList"])
        assert np.array_equal(got["pp"].cpu().numpy(), want["partPointer"])


@pytest.mark.parametrize("dim", [16, 22])
def test_forward_aggregation_matches_float64_on_every_row(prepared, cuda, dim):
    P = prepared
    n = P["n"]
    rng = np.random.Generator(np.random.PCG64(dim))
    feat = rng.standard_normal((n, dim)).astype(np.float32)
    want = O.spmm_forward(P["ip"], P["ix"], P["deg"], feat)
    ld = (dim + 7) // 8 * 8
    plain = torch.zeros(n, ld, device=cuda)[:, :dim]
    plain.copy_(t(feat, cuda))
    got = capi.spmm_forward(plain, P["row"], P["col"], P["degd"], P["pp"], P["p2n"], P["part"])
    assert_close(got.cpu().numpy(), want, what=f"group kernel, forward dim {dim}")
    scaled = plain * P["degd"][:, None]                                  # what the update step hands over
    got = capi.spmm_forward(scaled, P["row"], P["col"], P["degd"], P["pp"], P["p2n"], P["part"], prescaled=True)
    assert_close(got.cpu().numpy(), want, 2e-5, 2e-6, what=f"group kernel, pre-scaled rows, forward dim {dim}")
    src = torch.zeros(n, ld, device=cuda)[:, :dim]
    src.copy_(scaled)
    got = capi.spmm_tiles(src, capi.TilePlan.from_csr(P["row"], P["col"]), P["degd"])
    assert_close(got.cpu().numpy(), want, 2e-5, 2e-6, what=f"tiled kernel, forward dim {dim}")


@pytest.mark.parametrize("conv,dim", [(1, 22), (0, 16)])
def test_compacted_backward_matches_float64_on_every_row(prepared, cuda, conv, dim):
    P = prepared
    n = P["n"]
    p, w = P["path"][conv], P["want"][conv]
    rng = np.random.Generator(np.random.PCG64(100 + dim))
    d_out = rng.standard_normal((n, dim)).astype(np.float32)
    want = O.ours_backward_aggregate(w["id"], w["partPointer"], w["edgeList"], P["deg"], d_out, w["numParts"])
    dd = t(d_out, cuda)
    got = capi.spmm_backward_compacted(dd, p["id"], p["pp"], p["edges"], P["degd"], p["parts"], BACK)
    assert_close(got.cpu().numpy(), want, what=f"group kernel, backward conv {conv + 1}")
    ld = (dim + 7) // 8 * 8
    src = torch.zeros(n, ld, device=cuda)[:, :dim]
    src.copy_(dd * P["degd"][:, None])
    got = capi.spmm_tiles(src, capi.TilePlan.from_ids(p["id"], p["edges"], p["valid"], n), P["degd"])
    got = got.cpu().numpy()
    assert_close(got, want, 2e-5, 2e-6, what=f"tiled kernel, backward conv {conv + 1}")
    assert np.all(got[w["node_degs"] == 0] == 0), "rows off the path must come back zero"
