"""The operator module (GNNAdvisor API) and the autograd layer on a GPU,
against the float64 oracle and the golden vectors of the reference."""
import os

import numpy as np
import pytest
import torch

import eppgcn_b200
from eppgcn_b200 import graphs
from oracle import epp_oracle as O
from tests.golden import make_golden as G
from tests.helpers import assert_close, t

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gpu_ops.npz")


@pytest.fixture(scope="module")
def gnna():
    return eppgcn_b200.load_gnnadvisor()


def prepare_with_module(gnna, g, cuda, layers, part, back):
    n, e = len(g["indptr"]) - 1, len(g["indices"])
    pp, p2n = gnna.build_part(part, torch.from_numpy(g["indptr"]))
    pp, p2n = pp.int().to(cuda), p2n.int().to(cuda)
    col = t(g["indices"], cuda)
    ngh = [torch.zeros(n, dtype=torch.bool, device=cuda) for _ in range(layers - 1)]
    ems = [torch.full((e,), -1, dtype=torch.int32, device=cuda) for _ in range(layers)]
    nds = [torch.zeros(n, dtype=torch.int32, device=cuda) for _ in range(layers)]
    empty = torch.zeros(0, dtype=torch.bool, device=cuda)
    for i in range(layers):
        src = t(g["train"], cuda) if i == 0 else ngh[i - 1]
        dst = ngh[i] if i < layers - 1 else empty
        gnna.mask_forward(p2n, pp, col, src, dst, ems[layers - 1 - i], nds[layers - 1 - i], layers, i + 1, 4, 16)
    return pp, p2n, col, ngh, ems, nds


def test_module_reproduces_reference_golden_vectors(gnna, cuda):
    """Same seeded inputs as the stored outputs of the reference's CUDA
    operators: integer results bit-exact, float results within tolerance."""
    if not os.path.exists(GOLDEN):
        pytest.skip("ref_gpu_ops.npz has not been generated")
    z = np.load(GOLDEN)
    g = G.golden_inputs()
    L, e = G.GPU_LAYERS, len(g["indices"])
    pp, p2n, col, ngh, ems, nds = prepare_with_module(gnna, g, cuda, L, G.GPU_PART, G.GPU_BACK)
    row = t(g["indptr"], cuda)
    for i in range(L - 1):
        assert np.array_equal(ngh[i].cpu().numpy(), z[f"ngh_mask_{i}"])
    paths = []
    for i in range(L):
        assert np.array_equal(ems[i].cpu().numpy(), z[f"edge_mask_{i}"])
        assert np.array_equal(nds[i].cpu().numpy(), z[f"node_degs_{i}"])
        ids, edges, info = gnna.compact_back_edge(ems[i], col)
        assert int(info[0].item()) == int(z[f"valid_len_{i}"])
        assert np.array_equal(ids.cpu().numpy(), z[f"compact_id_{i}"])
        assert np.array_equal(edges.cpu().numpy(), z[f"compact_edge_{i}"])
        assert gnna.get_map_back_part_size(nds[i], int(info[0].item())) == int(z[f"map_size_{i}"])
        ppb, pinfo = gnna.split_back_part(nds[i], e, G.GPU_BACK)
        assert int(pinfo[0].item()) == int(z[f"num_parts_{i}"])
        assert np.array_equal(ppb.cpu().numpy()[:e], z[f"part_pointer_{i}"])
        bb = gnna.build_back_part(ems[i], col, nds[i], 0, 16)
        assert np.array_equal(bb[2].cpu().numpy()[:e], z[f"bbp_part_pointer_{i}"])
        np.testing.assert_array_equal(bb[3].numpy(), z[f"bbp_info_{i}"].astype(np.float64))
        paths.append((ids, ppb, edges, int(pinfo[0].item())))
    # Both sides are fp32 with different summation orders.  With the reference loader's sqrt(deg)
    # factors the terms of a sum reach 1e3..1e5 and cancel, so that convention is compared relative
    # to the largest magnitude of each result; the normalising convention keeps the strict bound.
    def check(got, want, strict, what):
        got, want = got.cpu().numpy(), np.asarray(want)
        s = 1.0 if strict else float(np.abs(want).max())
        assert_close(got / s, want / s, 2e-5, 2e-6 if strict else 1e-5, what)

    for conv in ("rsqrt", "sqrt"):
        strict = conv == "rsqrt"
        deg = t(g[f"deg_{conv}"], cuda)
        h = t(g["x"], cuda)
        for i in range(L):
            w = t(g["ws"][i], cuda)
            y = gnna.forward(h, w, row, col, deg, pp, p2n, G.GPU_PART, 16, 4)[0]
            check(y, z[f"forward_{conv}_{i}"], strict, f"forward {conv} {i}")
            ids, ppb, edges, nparts = paths[i]
            d_in, d_w = gnna.ours_backward(t(g["d_outs"][i], cuda), h, w, ids, ppb, edges, deg, G.GPU_BACK,
                                           nparts, i + 1, 4, 16)
            check(d_in, z[f"ours_backward_{conv}_{i}_dinput"], strict, "d_input")
            scale = float(np.abs(z[f"ours_backward_{conv}_{i}_dweight"]).max())
            assert_close(d_w.cpu().numpy() / scale, z[f"ours_backward_{conv}_{i}_dweight"] / scale, 1e-4, 1e-5,
                         "d_weight")
            d_in, _ = gnna.backward(t(g["d_outs"][i], cuda), h, w, row, col, deg, pp, p2n, G.GPU_PART, 16, 4)
            check(d_in, z[f"backward_{conv}_{i}_dinput"], strict, "backward")
            h = torch.relu(t(z[f"forward_{conv}_{i}"], cuda))


@pytest.mark.parametrize("workload", ["cora", "pubmed"])
def test_operators_against_float64_oracle(gnna, cuda, workload):
    ds = graphs.load_workload(workload, 0)
    ip, ix = ds.graph.indptr, ds.graph.indices
    n, e = ds.num_nodes, ds.num_edges
    part = int(ds.avg_degree)
    g = dict(indptr=ip, indices=ix, train=ds.train_mask.numpy())
    pp, p2n, col, ngh, ems, nds = prepare_with_module(gnna, g, cuda, 2, part, 32)
    want, _ = O.prepare_execution_path(ip, ix, g["train"], 2, part, [32, 32])
    rng = np.random.Generator(np.random.PCG64(5))
    x = rng.standard_normal((n, 96)).astype(np.float32)
    dims = [16, 22]
    ws = [rng.uniform(-0.25, 0.25, (96, 16)).astype(np.float32), rng.uniform(-0.2, 0.2, (16, 22)).astype(np.float32)]
    deg = ds.degrees.numpy()
    h = x
    for i in range(2):
        ids, edges, info = gnna.compact_back_edge(ems[i], col)
        ppb, pinfo = gnna.split_back_part(nds[i], e, 32)
        w = want[i]
        assert int(info[0].item()) == w["valid_len"] and int(pinfo[0].item()) == w["numParts"]
        assert np.array_equal(ids.cpu().numpy(), w["id"]) and np.array_equal(edges.cpu().numpy(), w["edgeList"])
        assert np.array_equal(ppb.cpu().numpy(), w["partPointer"])
        y = gnna.forward(t(h, cuda), t(ws[i], cuda), t(ip, cuda), col, t(deg, cuda), pp, p2n, part, 16, 8)[0]
        assert y.shape == (n, dims[i]) and y.is_contiguous()
        assert_close(y.cpu().numpy(), O.gcn_layer_forward(h, ws[i], ip, ix, deg), 2e-5, 2e-6, f"forward {i}")
        d_out = rng.standard_normal((n, dims[i])).astype(np.float32)
        d_in, d_w = gnna.ours_backward(t(d_out, cuda), t(h, cuda), t(ws[i], cuda), ids, ppb, edges, t(deg, cuda),
                                       32, int(pinfo[0].item()), i + 1, 4, 16)
        wi, ww, _ = O.gcn_layer_backward(d_out, h, ws[i], w["id"], w["partPointer"], w["edgeList"], deg,
                                         w["numParts"])
        assert_close(d_in.cpu().numpy(), wi, 2e-5, 2e-6, "d_input")
        s = float(np.abs(ww).max())
        assert_close(d_w.cpu().numpy() / s, ww / s, 1e-4, 1e-5, "d_weight")
        h = np.maximum(y.cpu().numpy(), 0)


def test_training_matches_dense_float64_autograd(cuda):
    """Two epochs of the harness on the Cora-shaped workload: loss and both
    weight gradients equal a dense float64 autograd GCN on the CPU."""
    from eppgcn_b200.train import GCNTrainer
    ds = graphs.load_workload("cora", 0)
    ip, ix = ds.graph.indptr.astype(np.int64), ds.graph.indices.astype(np.int64)
    n = ds.num_nodes
    deg = ds.degrees.double()
    rows = torch.from_numpy(np.repeat(np.arange(n), np.diff(ip)))
    a = torch.zeros(n, n, dtype=torch.float64)
    a[rows, torch.from_numpy(ix)] = 1.0
    a = deg[:, None] * a * deg[None, :]
    x64, y, train = ds.x.double(), ds.y.clone(), ds.train_mask.clone()
    tr = GCNTrainer(ds, hidden=16, backsize_mode="constant", backsize=32, prepare_before_training=False, seed=3)
    w = [p.detach().cpu().double().requires_grad_(True) for p in tr.model.parameters()]
    for epoch in range(2):
        loss = tr.train_epoch(isFirstIter=(epoch == 0))
        grads = [p.grad.detach().cpu().double() for p in tr.model.parameters()]
        h = torch.relu(a @ (x64 @ w[0]))
        out = a @ (h @ w[1])
        ref_loss = torch.nn.functional.nll_loss(torch.log_softmax(out, 1)[train], y[train])
        ref_grads = torch.autograd.grad(ref_loss, w)
        assert abs(loss.item() - ref_loss.item()) <= 1e-5 * max(1.0, abs(ref_loss.item()))
        for got, want in zip(grads, ref_grads):
            s = float(want.abs().max())
            assert_close(got.numpy() / s, want.numpy() / s, 1e-4, 1e-5, f"weight gradient, epoch {epoch}")
        with torch.no_grad():                         # follow the optimiser's fp32 weights
            w = [p.detach().cpu().double().requires_grad_(True) for p in tr.model.parameters()]
    assert tr.prepared and all(b.numParts > 0 for b in tr.back_props)


def test_timers_print_the_reference_keys(gnna, cuda, capfd):
    from eppgcn_b200.train import GCNTrainer
    ds = graphs.load_workload("cora", 0)
    tr = GCNTrainer(ds, prepare_before_training=False)
    tr.train_epoch(True)
    gnna.clear_time()
    for _ in range(3):
        tr.train_epoch(False)
    gnna.print_time()
    out = capfd.readouterr().out
    keys = [line.split(":")[0] for line in out.strip().splitlines()]
    assert keys == ["for_agg_time", "back_agg_time", "l1_back_agg_time", "l2_back_agg_time", "mask_time"]
    vals = {line.split(":")[0]: float(line.split(":")[1]) for line in out.strip().splitlines()}
    assert vals["for_agg_time"] > 0 and vals["back_agg_time"] > 0
    assert abs(vals["l1_back_agg_time"] + vals["l2_back_agg_time"] - vals["back_agg_time"]) < 1e-4
    assert vals["mask_time"] > 0      # clear_time leaves mask_time alone, EPPGCN_kernel.cu:108-116


def test_trainer_reads_a_prepared_path_back_from_disk(cuda, tmp_path):
    """Two trainers on the same workload and seed: the first prepares the path
    and writes it, the second loads it and must take exactly the same first step."""
    from tests.helpers import cached_path_scenario
    cached_path_scenario(tmp_path, "cuda")
