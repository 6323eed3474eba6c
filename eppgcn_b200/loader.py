"""Graph files of the reference's loader (EPPGCN/dataset.py:52-142).

Two formats, chosen by ``--loadFromTxt`` in the reference's script
(EPPGCN/gcn_main.py:73-78):

* ``<dataDir>/<name>_snap``: a text edge list, one ``src dst`` pair per line;
  the vertex count is the largest id + 1 (EPPGCN/dataset.py:56-73);
* ``<dataDir>/<name>.npz``: arrays ``src_li``, ``dst_li`` and the scalar
  ``num_nodes`` (EPPGCN/dataset.py:79-91);

plus ``<dataDir>/train_mask_<ratio>`` (``train_mask`` for ratio 0.0), one 0/1
value per line (EPPGCN/dataset.py:46-49).

The CSR is the one ``scipy.sparse.coo_matrix(...).tocsr()`` gives the reference
(EPPGCN/dataset.py:106-113): directed edges exactly as listed (no mirroring, no
self loops added), repeated pairs merged, columns sorted -- built here with one
numpy sort instead of a Python loop over the lines.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from .graphs import Graph, SyntheticDataset


def read_edge_list_txt(path: str):
    """``(src, dst, num_nodes)`` of a whitespace-separated edge list."""
    flat = np.fromfile(path, dtype=np.int64, sep=" ")
    if flat.size % 2:
        raise ValueError(f"{path}: odd number of integers, expected 'src dst' pairs")
    pairs = flat.reshape(-1, 2)
    if pairs.size and pairs.min() < 0:
        raise ValueError(f"{path}: negative vertex id")
    n = int(pairs.max()) + 1 if pairs.size else 0
    return pairs[:, 0].copy(), pairs[:, 1].copy(), n


def read_edge_list_npz(path: str):
    if not path.endswith(".npz"):
        raise ValueError("graph file must be a .npz file")           # EPPGCN/dataset.py:80-81
    with np.load(path) as obj:
        src, dst = np.asarray(obj["src_li"], dtype=np.int64), np.asarray(obj["dst_li"], dtype=np.int64)
        n = int(obj["num_nodes"])
    if src.shape != dst.shape:
        raise ValueError(f"{path}: src_li and dst_li differ in length")
    if src.size and (min(src.min(), dst.min()) < 0 or max(src.max(), dst.max()) >= n):
        raise ValueError(f"{path}: vertex id outside [0, num_nodes)")
    return src, dst, n


def csr_from_directed(num_nodes: int, src: np.ndarray, dst: np.ndarray):
    """Row = ``src``, column = ``dst``; repeated pairs merged, columns sorted."""
    if num_nodes >= 2**31 or src.size >= 2**31:
        raise ValueError("graph does not fit int32 indexing")
    key = np.unique(src.astype(np.int64) * num_nodes + dst.astype(np.int64)) if src.size else np.zeros(0, np.int64)
    rows = key // max(num_nodes, 1)
    indptr = np.zeros(num_nodes + 1, dtype=np.int64)
    np.cumsum(np.bincount(rows, minlength=num_nodes), out=indptr[1:])
    return indptr.astype(np.int32), (key - rows * num_nodes).astype(np.int32)


def read_train_mask(data_dir: str, ratio: float, num_nodes: int) -> np.ndarray:
    name = "train_mask" if ratio == 0.0 else "train_mask_" + str(ratio)
    mask = np.atleast_1d(np.genfromtxt(os.path.join(data_dir, name), delimiter="\n"))
    if mask.shape[0] != num_nodes:
        raise ValueError(f"{name}: {mask.shape[0]} entries for {num_nodes} vertices")
    return mask != 0


class FileDataset(SyntheticDataset):
    """The reference's ``custom_dataset`` (EPPGCN/dataset.py:18-156) with the
    same constructor arguments and attributes, tensors on ``device``.

    Differences, both on the safe side: ``num_edges`` is the number of stored
    CSR entries (the reference keeps the raw line count, which is larger when
    the file repeats a pair, and sizes its edge masks by it), while
    ``avg_degree`` and ``avg_edgeSpan`` follow the raw list as in the reference
    (EPPGCN/dataset.py:93-94) because the group size is derived from them.
    ``degrees`` holds ``sqrt(max(deg, 1))`` as the reference loader does
    (EPPGCN/dataset.py:118-119) unless ``degree_norm="rsqrt"`` is asked for.
    """

    def __init__(self, path, dataPath, ratio, dim, num_class, num_layer, load_from_txt=True, verbose=False,
                 degree_norm: str = "sqrt", seed: int = 0, device="cpu"):
        src, dst, n = read_edge_list_txt(path) if load_from_txt else read_edge_list_npz(path)
        indptr, indices = csr_from_directed(n, src, dst)
        graph = Graph(indptr, indices, name=os.path.basename(path), seed=seed)
        super().__init__(graph, dim, num_class, num_layer, train_ratio=0.0, x_kind="normal", seed=seed,
                         degree_norm=degree_norm, device="cpu")
        raw = int(src.shape[0])
        self.avg_degree = raw / n if n else 0.0
        self.avg_edgeSpan = float(np.mean(np.abs(src - dst))) if raw else 0.0
        self.train_mask = torch.from_numpy(read_train_mask(dataPath, ratio, n))
        val, test = 0.3, 0.1                                            # EPPGCN/dataset.py:136-139
        ar = torch.arange(n)
        self.val_mask, self.test_mask = ar < int(n * val), ar < int(n * test)
        if verbose:
            print("# nodes: {}".format(n))
            print("# avg_degree: {:.2f}".format(self.avg_degree))
            print("# avg_edgeSpan: {}".format(int(self.avg_edgeSpan)))
        self.reset_masks()
        self.to(device)

    def to(self, device):
        super().to(device)
        for k in ("val_mask", "test_mask"):
            if hasattr(self, k):
                setattr(self, k, getattr(self, k).to(device))
        return self


def load_dataset_files(data_dir: str, name: str, ratio: float, dim: int, num_class: int, num_layer: int,
                       load_from_txt: bool = True, **kw) -> FileDataset:
    """File names as the reference's script composes them (EPPGCN/gcn_main.py:73-78)."""
    path = os.path.join(data_dir, name + "_snap") if load_from_txt else os.path.join(data_dir, name + ".npz")
    return FileDataset(path, data_dir, ratio, dim, num_class, num_layer, load_from_txt=load_from_txt, **kw)
