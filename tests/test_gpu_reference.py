"""Side by side with the reference's own CUDA operators (the unmodified
extension under oracle/_ref) on identical seeded inputs.  Integer metadata
must be bit-exact; aggregations within the float tolerance."""
import numpy as np
import pytest
import torch

import eppgcn_b200
from eppgcn_b200 import graphs
from oracle import epp_oracle as O
from oracle.ref_loader import load_reference
from tests.helpers import assert_close, t

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def both():
    ref = load_reference()
    if ref is None:
        pytest.skip("oracle/_ref holds no reference build")
    return eppgcn_b200.load_gnnadvisor(), ref


@pytest.mark.parametrize("workload,back", [("cora", 4), ("pubmed", 32), ("rmat16", 32), ("rmat19", 32)])
def test_preparation_and_operators_match_the_reference(both, cuda, workload, back):
    ours, ref = both
    ds = graphs.load_workload(workload, 0)
    n, e, L = ds.num_nodes, ds.num_edges, 2
    part = int(ds.avg_degree)
    ip = ds.row_pointers
    assert ds.graph.indptr[-1] > ds.graph.indptr[-2] and e < 2 ** 24     # inside the reference's build_part range
    po, no = ours.build_part(part, ip)
    if e < 2_000_000:        # the reference fills its outputs element by element: minutes beyond this size
        pr, nr = ref.build_part(part, ip)
        assert torch.equal(pr.int(), po) and torch.equal(nr.int(), no)
    pp, p2n = po.to(cuda), no.to(cuda)
    row, col, deg = ip.to(cuda), ds.column_index.to(cuda), ds.degrees.to(cuda)
    train = ds.train_mask.to(cuda)

    def prepare(mod):
        ngh = [torch.zeros(n, dtype=torch.bool, device=cuda) for _ in range(L - 1)]
        ems = [torch.full((e,), -1, dtype=torch.int32, device=cuda) for _ in range(L)]
        nds = [torch.zeros(n, dtype=torch.int32, device=cuda) for _ in range(L)]
        empty = torch.zeros(0, dtype=torch.bool, device=cuda)
        for i in range(L):
            mod.mask_forward(p2n, pp, col, train if i == 0 else ngh[i - 1], ngh[i] if i < L - 1 else empty,
                             ems[L - 1 - i], nds[L - 1 - i], L, i + 1, 4, 16)
        return ngh, ems, nds

    (ngh_o, ems_o, nds_o), (ngh_r, ems_r, nds_r) = prepare(ours), prepare(ref)
    g = torch.Generator(device=cuda).manual_seed(1)
    h = torch.randn(n, ds.num_features, device=cuda, generator=g)
    dims = [16, 22]
    for i in range(L):
        assert torch.equal(ems_o[i], ems_r[i]) and torch.equal(nds_o[i], nds_r[i])
        if i < L - 1:
            assert torch.equal(ngh_o[i], ngh_r[i])
        io, eo, vo = ours.compact_back_edge(ems_o[i], col)
        ir, er, vr = ref.compact_back_edge(ems_r[i], col)
        assert int(vo[0].item()) == int(vr[0].item()) and torch.equal(io, ir) and torch.equal(eo, er)
        assert ours.get_map_back_part_size(nds_o[i], int(vo[0].item())) == \
            ref.get_map_back_part_size(nds_r[i], int(vr[0].item()))
        so, co = ours.split_back_part(nds_o[i], e, back)
        nparts = int(co[0].item())
        if O.split_reference_valid(nds_o[i].cpu().numpy(), back):
            sr, cr = ref.split_back_part(nds_r[i], e, back)
            assert int(cr[0].item()) == nparts and torch.equal(so[:e], sr)
        w = (torch.rand(h.size(1), dims[i], device=cuda, generator=g) - 0.5) / 2
        yo = ours.forward(h, w, row, col, deg, pp, p2n, part, 16, 8)[0]
        yr = ref.forward(h, w, row, col, deg, pp, p2n, part, 16, 8)[0]
        assert_close(yo.cpu().numpy(), yr.cpu().numpy(), 2e-5, 2e-6, f"forward {i}")
        d_out = torch.randn(n, dims[i], device=cuda, generator=g)
        do, wo = ours.ours_backward(d_out, h, w, io, so, eo, deg, back, nparts, i + 1, 4, 16)
        dr, wr = ref.ours_backward(d_out, h, w, io, so, eo, deg, back, nparts, i + 1, 4, 16)
        assert_close(do.cpu().numpy(), dr.cpu().numpy(), 2e-5, 2e-6, f"d_input {i}")
        s = float(wr.abs().max())
        assert_close((wo / s).cpu().numpy(), (wr / s).cpu().numpy(), 1e-4, 1e-5, f"d_weight {i}")
        do, _ = ours.backward(d_out, h, w, row, col, deg, pp, p2n, part, 16, 8)
        dr, _ = ref.backward(d_out, h, w, row, col, deg, pp, p2n, part, 16, 8)
        assert_close(do.cpu().numpy(), dr.cpu().numpy(), 2e-5, 2e-6, f"backward {i}")
        h = torch.relu(yr)
