"""The training harness on the CPU, with the operator module replaced by a
numpy double built from the oracle: call order, first-iteration preparation,
part-size rules, gradients through the autograd boundary, and the on-disk
cache of prepared paths.  The operators themselves are checked on GPUs."""
import types

import numpy as np
import pytest
import torch

from oracle import epp_oracle as O
from tests.helpers import cached_path_scenario


def _operator_double(real):
    """Same twelve names and return shapes as the operator module, CPU tensors."""
    def t32(a):
        return torch.from_numpy(np.asarray(a, dtype=np.int32))

    def forward(X, W, row_pointers, column_index, degrees, partPtr, part2Node, partSize, dimWorker, warpPerBlock):
        out = O.spmm_forward(row_pointers.numpy(), column_index.numpy(), degrees.numpy(),
                             (X.double() @ W.double()).numpy())
        return [torch.from_numpy(out.astype(np.float32))]

    def ours_backward(d_output, X, W, ids, partPointer, edgeList, degrees, partSize, numParts, layer, blockx, blocky):
        d_prime = O.ours_backward_aggregate(ids.numpy(), partPointer.numpy(), edgeList.numpy(), degrees.numpy(),
                                            d_output.numpy(), numParts)
        d_prime = torch.from_numpy(d_prime)
        return [(d_prime @ W.double().T).float(), (X.double().T @ d_prime).float()]

    def mask_forward(ids, partPointer, edgeList, src_mask, ngh_mask, backEdgeMask, node_degs, num_layers, layer,
                     blockx, blocky):
        O.mask_forward(ids.numpy(), partPointer.numpy(), edgeList.numpy(), src_mask.numpy(), ngh_mask.numpy(),
                       backEdgeMask.numpy(), node_degs.numpy(), num_layers, layer)

    def compact_back_edge(edge_mask, column_index):
        ids, cols, valid = O.compact_back_edge(edge_mask.numpy(), column_index.numpy())
        return [t32(ids), t32(cols), torch.tensor([float(valid)], dtype=torch.float64)]

    def split_back_part(node_deg, num_edges, part_size):
        pp, parts = O.split_back_part(node_deg.numpy(), num_edges, part_size, out_len=num_edges + 1)
        return [t32(pp), torch.tensor([int(parts)], dtype=torch.int32)]

    return types.SimpleNamespace(
        forward=forward, ours_backward=ours_backward, mask_forward=mask_forward,
        compact_back_edge=compact_back_edge, split_back_part=split_back_part,
        get_map_back_part_size=lambda node_deg, valid_len: O.get_map_back_part_size(node_deg.numpy(), valid_len),
        build_part=real.build_part, print_time=lambda: None, clear_time=lambda: None)


@pytest.fixture
def cpu_operators(monkeypatch):
    from eppgcn_b200 import gcn_conv, train
    double = _operator_double(train.GNNA)
    monkeypatch.setattr(train, "GNNA", double)
    monkeypatch.setattr(gcn_conv, "GNNA", double)
    return double


def test_first_iteration_prepares_the_path_and_training_reduces_the_loss(cpu_operators):
    from eppgcn_b200 import graphs
    from eppgcn_b200.train import GCNTrainer
    ds = graphs.load_workload("cora", 0)
    tr = GCNTrainer(ds, hidden=16, backsize_mode="bucket", prepare_before_training=False, seed=1, device="cpu")
    assert not tr.prepared
    losses = [float(tr.train_epoch(i == 0).item()) for i in range(6)]
    assert tr.prepared and all(p.numParts > 0 and p.partSize in (4, 8, 16, 32, 64) for p in tr.back_props)
    assert losses[-1] < losses[0]
    want, _ = O.prepare_execution_path(ds.graph.indptr, ds.graph.indices, ds.train_mask.numpy(), 2,
                                       tr.inputInfo.partSize, [p.partSize for p in tr.back_props])
    for got, ref in zip(tr.back_props, want):
        assert got.valid_len == ref["valid_len"] and got.numParts == ref["numParts"]
        assert np.array_equal(got.id.numpy()[:got.valid_len], ref["id"][:ref["valid_len"]])


def test_preparing_before_training_gives_the_same_path(cpu_operators):
    from eppgcn_b200 import graphs
    from eppgcn_b200.train import GCNTrainer
    early = GCNTrainer(graphs.load_workload("cora", 0), backsize_mode="constant", backsize=8,
                       prepare_before_training=True, seed=1, device="cpu")
    late = GCNTrainer(graphs.load_workload("cora", 0), backsize_mode="constant", backsize=8,
                      prepare_before_training=False, seed=1, device="cpu")
    late.train_epoch(True)
    for a, b in zip(early.back_props, late.back_props):
        assert a.numParts == b.numParts and torch.equal(a.id, b.id) and torch.equal(a.partPointer, b.partPointer)


def test_prepared_path_is_read_back_from_disk(cpu_operators, tmp_path):
    first, second = cached_path_scenario(tmp_path, "cpu")
    assert second.build_time >= 0.0


def test_harness_runs_on_a_graph_read_from_files(cpu_operators, tmp_path):
    """The reference's file layout (edge list + train mask) through the loader and the harness."""
    from eppgcn_b200 import loader
    from eppgcn_b200.train import GCNTrainer
    rng = np.random.Generator(np.random.PCG64(4))
    n = 150
    src, dst = rng.integers(0, n, 900), rng.integers(0, n, 900)
    src, dst = np.concatenate([src, dst, [n - 1]]), np.concatenate([dst, src, [n - 1]])     # symmetric, ids up to n-1
    with open(tmp_path / "toy_snap", "w") as f:
        f.writelines(f"{s} {d}\n" for s, d in zip(src, dst))
    np.savetxt(tmp_path / "train_mask_0.3", (rng.random(n) < 0.3).astype(int), fmt="%d")
    ds = loader.load_dataset_files(str(tmp_path), "toy", 0.3, 12, 5, 2, degree_norm="rsqrt")
    tr = GCNTrainer(ds, hidden=8, backsize_mode="map", prepare_before_training=False, seed=2, device="cpu")
    losses = [float(tr.train_epoch(i == 0).item()) for i in range(5)]
    assert tr.prepared and np.isfinite(losses).all() and losses[-1] < losses[0]
    assert tr.inputInfo.partSize == max(int(ds.avg_degree), 1)
