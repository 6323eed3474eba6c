"""File loader against what the reference's loader computes (scipy COO -> CSR,
EPPGCN/dataset.py:106-119) on small edge lists written to a temporary folder."""
import numpy as np
import pytest
import torch
from scipy.sparse import coo_matrix

from eppgcn_b200 import loader


def _write(tmp_path, src, dst, n, ratio=0.1, seed=0):
    with open(tmp_path / "toy_snap", "w") as f:
        for s, d in zip(src, dst):
            f.write(f"{s}\t{d}\n")
    np.savez(tmp_path / "toy.npz", src_li=np.asarray(src), dst_li=np.asarray(dst), num_nodes=n)
    mask = (np.random.Generator(np.random.PCG64(seed)).random(n) < ratio).astype(int)
    np.savetxt(tmp_path / f"train_mask_{ratio}", mask, fmt="%d")
    np.savetxt(tmp_path / "train_mask", 1 - mask, fmt="%d")
    return mask.astype(bool)


def _reference_csr(src, dst, n):
    csr = coo_matrix(([1] * len(src), np.stack([src, dst])), shape=(n, n)).tocsr()
    return csr.indptr.astype(np.int32), csr.indices.astype(np.int32)


@pytest.mark.parametrize("from_txt", [True, False])
def test_matches_the_scipy_csr_of_the_reference_loader(tmp_path, from_txt):
    rng = np.random.Generator(np.random.PCG64(3))
    n = 200
    src = rng.integers(0, n - 1, 1500)            # vertex n-2 .. has no out-edges; repeated pairs are likely
    dst = rng.integers(0, n, 1500)
    dst[0], src[0] = n - 1, 0                     # the largest id fixes the vertex count of the text format
    src, dst = np.concatenate([src, src[:40]]), np.concatenate([dst, dst[:40]])      # certain repeats
    mask = _write(tmp_path, src, dst, n)
    ds = loader.load_dataset_files(str(tmp_path), "toy", 0.1, 12, 5, 3, load_from_txt=from_txt)
    indptr, indices = _reference_csr(src, dst, n)
    assert np.array_equal(ds.row_pointers.numpy(), indptr) and np.array_equal(ds.column_index.numpy(), indices)
    assert ds.row_pointers.dtype == torch.int32 and ds.column_index.dtype == torch.int32
    assert ds.num_nodes == n and ds.num_edges == len(indices)
    assert ds.avg_degree == len(src) / n                                   # raw line count, as the reference
    assert ds.avg_edgeSpan == pytest.approx(np.mean(np.abs(src - dst)))
    deg = np.maximum(np.diff(indptr), 1)
    assert np.allclose(ds.degrees.numpy(), np.sqrt(deg).astype(np.float32))
    assert np.array_equal(ds.train_mask.numpy(), mask)
    assert ds.x.shape == (n, 12) and ds.y.dtype == torch.long and bool((ds.y == 1).all())
    assert len(ds.ngh_masks) == 2 and len(ds.edge_masks) == 3 and ds.edge_masks[0].numel() == ds.num_edges
    assert int(ds.val_mask.sum()) == int(n * 0.3) and int(ds.test_mask.sum()) == int(n * 0.1)
    other = loader.load_dataset_files(str(tmp_path), "toy", 0.0, 12, 5, 3, load_from_txt=from_txt)
    assert np.array_equal(other.train_mask.numpy(), ~mask)                 # ratio 0.0 reads `train_mask`


def test_rejects_broken_files(tmp_path):
    (tmp_path / "odd_snap").write_text("0 1\n2\n")
    with pytest.raises(ValueError):
        loader.read_edge_list_txt(str(tmp_path / "odd_snap"))
    with pytest.raises(ValueError):
        loader.read_edge_list_npz(str(tmp_path / "graph.txt"))
    np.savez(tmp_path / "bad.npz", src_li=np.array([0, 5]), dst_li=np.array([1, 2]), num_nodes=3)
    with pytest.raises(ValueError):
        loader.read_edge_list_npz(str(tmp_path / "bad.npz"))
    _write(tmp_path, [0, 1], [1, 0], 2)
    np.savetxt(tmp_path / "train_mask_0.5", np.array([1, 0, 1]), fmt="%d")
    with pytest.raises(ValueError):
        loader.load_dataset_files(str(tmp_path), "toy", 0.5, 4, 2, 2)


def test_empty_rows_and_single_vertex(tmp_path):
    indptr, indices = loader.csr_from_directed(4, np.array([3, 3, 0]), np.array([2, 2, 0]))
    assert indptr.tolist() == [0, 1, 1, 1, 2] and indices.tolist() == [0, 2]
    indptr, indices = loader.csr_from_directed(1, np.zeros(0, np.int64), np.zeros(0, np.int64))
    assert indptr.tolist() == [0, 0] and indices.size == 0
