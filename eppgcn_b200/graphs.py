"""Seeded synthetic graphs and the dataset bag the GCN hot path consumes.

The reference trains on public SNAP / npz graphs with train-mask text files
(EPPGCN/dataset.py:52-119, :45-48).  None of those files ship with it, so the
workloads here are seeded generators with the same shapes: a Chung-Lu
power-law model for the citation/social shaped graphs and R-MAT for the large
ones.  Every graph is symmetrised, de-duplicated, stripped of self edges and
then given exactly one self loop per vertex; the CSR has int32 indices and
sorted columns, which is what ``scipy.sparse.coo_matrix(...).tocsr()`` hands
the reference (EPPGCN/dataset.py:105-115).

``SyntheticDataset`` carries the same attributes as the reference's
``custom_dataset`` (EPPGCN/dataset.py:18-156): ``row_pointers``/``column_index``
(CPU int32), ``degrees`` (fp32), ``x``, ``y``, ``train_mask``, the per-layer
``ngh_masks`` (bool[N], zeros), ``edge_masks`` (int32[E], -1), ``node_degs``
(int32[N], zeros) and the empty mask used for the last preparation step.
"""
from __future__ import annotations

import hashlib
import os
from dataclasses import dataclass

import numpy as np
import torch

__all__ = [
    "Graph", "WORKLOADS", "make_graph", "chung_lu", "rmat", "csr_from_pairs",
    "SyntheticDataset", "load_workload",
]


@dataclass
class Graph:
    """CSR adjacency (int32, sorted columns, one self loop per vertex)."""
    indptr: np.ndarray      # int32[N+1]
    indices: np.ndarray     # int32[E]
    name: str = ""
    seed: int = 0

    @property
    def num_nodes(self) -> int:
        return int(self.indptr.shape[0] - 1)

    @property
    def num_edges(self) -> int:
        return int(self.indices.shape[0])


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def csr_from_pairs(n: int, src: np.ndarray, dst: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """Undirected pairs -> symmetric CSR with self loops.

    Mirrors each pair, drops duplicates and self edges, appends one self loop
    per vertex and sorts by (row, col) with a single key sort.
    """
    src = src.astype(np.int64, copy=False)
    dst = dst.astype(np.int64, copy=False)
    keep = src != dst
    src, dst = src[keep], dst[keep]
    loops = np.arange(n, dtype=np.int64)
    key = np.concatenate([src * n + dst, dst * n + src, loops * n + loops])
    key.sort()
    uniq = np.empty(key.shape[0], dtype=bool)
    uniq[0] = True
    np.not_equal(key[1:], key[:-1], out=uniq[1:])
    key = key[uniq]
    rows = key // n
    cols = (key - rows * n).astype(np.int32)
    counts = np.bincount(rows, minlength=n)
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(counts, out=indptr[1:])
    if indptr[-1] >= 2**31:
        raise ValueError("edge count exceeds int32 indexing")
    return indptr.astype(np.int32), cols


def _collect_unique_pairs(draw, n: int, target: int) -> np.ndarray:
    """Keys ``lo*n+hi`` of exactly ``target`` distinct undirected non-loop
    pairs.  ``draw(count)`` returns two endpoint arrays.  Batches are drawn
    until enough distinct pairs exist; the surplus is trimmed from the last
    batch in order of first appearance, so the result depends only on the seed."""
    have = np.empty(0, dtype=np.int64)          # sorted, distinct
    first = True
    while True:
        need = target - have.shape[0]
        if need <= 0:
            return have
        count = target if first else int(need * 1.25) + 4096
        first = False
        a, b = draw(count)
        lo, hi = np.minimum(a, b), np.maximum(a, b)
        key = (lo * n + hi)[lo != hi]
        order = np.argsort(key, kind="stable")
        sk = key[order]
        head = np.empty(sk.shape[0], dtype=bool)
        head[0] = True
        np.not_equal(sk[1:], sk[:-1], out=head[1:])
        sk, pos = sk[head], order[head]          # distinct keys, first position of each
        if have.shape[0]:
            at = np.searchsorted(have, sk)
            at[at == have.shape[0]] = have.shape[0] - 1
            fresh = have[at] != sk
            sk, pos = sk[fresh], pos[fresh]
        if sk.shape[0] > need:
            sel = np.argsort(pos, kind="stable")[:need]
            sk = sk[sel]
        have = np.concatenate([have, sk])
        have.sort()


def chung_lu(n: int, pairs: int, exponent: float, seed: int, offset: float = 10.0):
    """Exactly ``pairs`` distinct undirected non-loop pairs, endpoints drawn
    with probability proportional to ``(rank + offset) ** (-1/(exponent-1))``
    and then relabelled by a seeded permutation so hubs are spread over the
    id range (real graphs are not sorted by degree)."""
    rng = _rng(seed)
    w = (np.arange(n, dtype=np.float64) + offset) ** (-1.0 / (exponent - 1.0))
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    perm = rng.permutation(n).astype(np.int64)

    def draw(count):
        a = np.searchsorted(cdf, rng.random(count), side="right")
        b = np.searchsorted(cdf, rng.random(count), side="right")
        return np.minimum(a, n - 1), np.minimum(b, n - 1)

    key = _collect_unique_pairs(draw, n, pairs)
    return perm[key // n], perm[key % n]


def rmat(scale: int, pairs_per_vertex: int, a: float, b: float, c: float, seed: int):
    """R-MAT: exactly ``pairs_per_vertex * 2**scale`` distinct undirected
    non-loop pairs, one quadrant choice per bit level with probabilities
    (a, b, c, 1-a-b-c)."""
    rng = _rng(seed)
    n = 1 << scale
    ab, abc = a + b, a + b + c

    def draw(count):
        src = np.zeros(count, dtype=np.int64)
        dst = np.zeros(count, dtype=np.int64)
        for _ in range(scale):
            r = rng.random(count, dtype=np.float32)
            sbit = r >= ab                                  # quadrants c, d
            dbit = ((r >= a) & (r < ab)) | (r >= abc)       # quadrants b, d
            src = (src << 1) | sbit
            dst = (dst << 1) | dbit
        return src, dst

    key = _collect_unique_pairs(draw, n, pairs_per_vertex * n)
    return key // n, key % n


# name -> (generator spec, model shape).  Sizes follow the five benchmark
# configurations this hot path is quoted on.
WORKLOADS = {
    "cora":   dict(kind="chung_lu", n=2708, pairs=5278, exponent=2.7,
                   dim=96, hidden=16, classes=22, layers=2, train_ratio=0.1, x="ones"),
    "pubmed": dict(kind="chung_lu", n=19717, pairs=88648, exponent=2.7,
                   dim=96, hidden=16, classes=22, layers=2, train_ratio=0.1, x="ones"),
    "social": dict(kind="chung_lu", n=1_130_000, pairs=5_980_000, exponent=2.1,
                   dim=96, hidden=16, classes=22, layers=2, train_ratio=0.1, x="uniform"),
    "rmat21": dict(kind="rmat", scale=21, edge_factor=8, a=0.57, b=0.19, c=0.19,
                   dim=128, hidden=16, classes=22, layers=2, train_ratio=0.1, x="normal"),
    "rmat24": dict(kind="rmat", scale=24, edge_factor=16, a=0.57, b=0.19, c=0.19, draw="device",
                   dim=128, hidden=64, classes=32, layers=3, train_ratio=0.05, x="normal"),
    # the same 3-layer shape at a size that draws in a second (tests of the device-drawn path)
    "rmat18x3": dict(kind="rmat", scale=18, edge_factor=16, a=0.57, b=0.19, c=0.19, draw="device",
                     dim=128, hidden=64, classes=32, layers=3, train_ratio=0.05, x="normal"),
    # small R-MAT used by tests and profiler captures (same generator, fewer levels)
    "rmat16": dict(kind="rmat", scale=16, edge_factor=8, a=0.57, b=0.19, c=0.19,
                   dim=128, hidden=16, classes=22, layers=2, train_ratio=0.1, x="normal"),
    "rmat19": dict(kind="rmat", scale=19, edge_factor=8, a=0.57, b=0.19, c=0.19,
                   dim=128, hidden=16, classes=22, layers=2, train_ratio=0.1, x="normal"),
}
# "edge factor 16 / 33.5M edges symmetrised" at scale 21 is 2**24 distinct
# pairs mirrored into 33.55M directed edges, i.e. 8 pairs per vertex; scale 24
# with "edge factor 32 / ~537M directed" is 16 pairs per vertex.


def _cache_dir() -> str:
    d = os.environ.get("EPPGCN_B200_CACHE", "/tmp/eppgcn_b200_cache")
    os.makedirs(d, exist_ok=True)
    return d


def make_graph(name: str, seed: int = 0, cache: bool = True) -> Graph:
    """Generate (or load from the local cache) the CSR of a named workload."""
    spec = WORKLOADS[name]
    tag = hashlib.sha1(repr((name, sorted(spec.items()), seed, 2)).encode()).hexdigest()[:12]
    path = os.path.join(_cache_dir(), f"{name}_{seed}_{tag}.npz")
    if cache and os.path.exists(path):
        z = np.load(path)
        return Graph(z["indptr"], z["indices"], name, seed)
    if spec["kind"] == "chung_lu":
        s, d = chung_lu(spec["n"], spec["pairs"], spec["exponent"], seed)
        n = spec["n"]
    else:
        s, d = rmat(spec["scale"], spec["edge_factor"], spec["a"], spec["b"], spec["c"], seed)
        n = 1 << spec["scale"]
    indptr, indices = csr_from_pairs(n, s, d)
    if cache and indices.shape[0] > 1_000_000:
        tmp = path + f".{os.getpid()}.tmp.npz"
        np.savez(tmp, indptr=indptr, indices=indices)
        os.replace(tmp, path)
    return Graph(indptr, indices, name, seed)


class SyntheticDataset:
    """Attribute-compatible stand-in for the reference's ``custom_dataset``
    (EPPGCN/dataset.py:18-156) built from a generated :class:`Graph`.

    ``degree_norm``: ``"rsqrt"`` stores ``deg**-0.5`` so the operator's
    ``degrees[row] * degrees[col]`` edge weight is the symmetric GCN
    normalisation; ``"sqrt"`` reproduces the reference loader's
    ``sqrt(max(deg, 1))`` (EPPGCN/dataset.py:118-119).  The operator multiplies
    whatever it is given.
    """

    def __init__(self, graph: Graph, dim: int, num_classes: int, num_layers: int,
                 train_ratio: float, x_kind: str = "normal", seed: int = 0,
                 degree_norm: str = "rsqrt", device: str | torch.device = "cpu"):
        self.graph = graph
        self.num_nodes = graph.num_nodes
        self.num_edges = graph.num_edges
        self.num_features = dim
        self.num_classes = num_classes
        self.num_layers = num_layers
        self.avg_degree = self.num_edges / self.num_nodes
        rows = np.repeat(np.arange(self.num_nodes, dtype=np.int64), np.diff(graph.indptr))
        self.avg_edgeSpan = float(np.mean(np.abs(rows - graph.indices))) if self.num_edges else 0.0
        del rows
        self.row_pointers = torch.from_numpy(graph.indptr)      # CPU int32, as the loader leaves it
        self.column_index = torch.from_numpy(graph.indices)
        deg = np.maximum(np.diff(graph.indptr), 1).astype(np.float32)
        deg = 1.0 / np.sqrt(deg) if degree_norm == "rsqrt" else np.sqrt(deg)
        self.degrees = torch.from_numpy(deg.astype(np.float32))
        g = torch.Generator().manual_seed(seed + 1)
        if x_kind == "ones":
            self.x = torch.ones(self.num_nodes, dim)
        elif x_kind == "uniform":
            self.x = torch.rand(self.num_nodes, dim, generator=g)
        else:
            self.x = torch.randn(self.num_nodes, dim, generator=g)
        self.y = torch.ones(self.num_nodes, dtype=torch.long)
        rng = _rng(seed + 2)
        self.train_mask = torch.from_numpy(rng.random(self.num_nodes) < train_ratio)
        self.reset_masks()
        self.to(device)

    def reset_masks(self):
        """Fresh preparation state (EPPGCN/dataset.py:144-156)."""
        dev = self.train_mask.device
        L, N, E = self.num_layers, self.num_nodes, self.num_edges
        self.ngh_masks = [torch.zeros(N, dtype=torch.bool, device=dev) for _ in range(L - 1)]
        self.empty_mask = torch.zeros(0, dtype=torch.bool, device=dev)
        self.edge_masks = [torch.full((E,), -1, dtype=torch.int32, device=dev) for _ in range(L)]
        self.node_degs = [torch.zeros(N, dtype=torch.int32, device=dev) for _ in range(L)]

    def to(self, device):
        """Moves what the reference keeps on the GPU; the CSR stays on the
        host until ``build_part`` has read it (EPPGCN/gcn_main.py:120-128)."""
        for k in ("degrees", "x", "y", "train_mask", "empty_mask"):
            setattr(self, k, getattr(self, k).to(device))
        for k in ("ngh_masks", "edge_masks", "node_degs"):
            setattr(self, k, [t.to(device) for t in getattr(self, k)])
        return self


def load_workload(name: str, seed: int = 0, device="cpu", train_ratio: float | None = None,
                  degree_norm: str = "rsqrt", layers: int | None = None) -> SyntheticDataset:
    spec = WORKLOADS[name]
    g = make_graph(name, seed)
    ds = SyntheticDataset(g, spec["dim"], spec["classes"], layers or spec["layers"],
                          spec["train_ratio"] if train_ratio is None else train_ratio,
                          spec["x"], seed, degree_norm, device)
    ds.hidden = spec["hidden"]
    ds.name = name
    return ds


# ---------------------------------------------------------------------------
# Device-side generation for the workloads that are too large to draw on the
# host in reasonable time (R-MAT scale 24: 268 M pairs, 24 levels each).
# ---------------------------------------------------------------------------
def rmat_csr_device(scale: int, pairs_per_vertex: int, a: float, b: float, c: float, seed: int, device):
    """R-MAT CSR built on ``device``: ``pairs_per_vertex * 2**scale`` draws,
    mirrored, de-duplicated, self edges replaced by one self loop per vertex.
    Unlike the host generator the duplicate draws are not replaced, so the edge
    count is a little below the nominal one (as in Graph500).  The same seed on
    the same GPU model gives the same graph, so every rank can draw its own copy.
    Returns ``(indptr int32[N+1], indices int32[E])`` on the device."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    n = 1 << scale
    total = pairs_per_vertex * n
    ab, abc = a + b, a + b + c
    keys = []
    chunk = 1 << 26
    for start in range(0, total, chunk):
        m = min(chunk, total - start)
        src = torch.zeros(m, dtype=torch.int64, device=dev)
        dst = torch.zeros(m, dtype=torch.int64, device=dev)
        for _ in range(scale):
            r = torch.rand(m, device=dev, generator=gen)
            src = (src << 1) | (r >= ab)
            dst = (dst << 1) | (((r >= a) & (r < ab)) | (r >= abc))
        keep = src != dst
        src, dst = src[keep], dst[keep]
        keys.append(src * n + dst)
        keys.append(dst * n + src)
        del src, dst, keep, r
    loops = torch.arange(n, dtype=torch.int64, device=dev)
    keys.append(loops * n + loops)
    key = torch.cat(keys)
    del keys, loops
    key = torch.unique(key)                       # sorted, distinct (row-major order)
    if key.numel() >= 2 ** 31:
        raise ValueError("edge count exceeds int32 indexing")
    rows = key >> scale
    indices = (key & (n - 1)).to(torch.int32)
    del key
    counts = torch.bincount(rows, minlength=n)
    del rows
    indptr = torch.zeros(n + 1, dtype=torch.int64, device=dev)
    torch.cumsum(counts, 0, out=indptr[1:])
    return indptr.to(torch.int32), indices


class DeviceWorkload:
    """A workload whose graph lives on the GPU from the start: the fields the
    hot path needs, named as in :class:`SyntheticDataset`."""

    def __init__(self, name: str, seed: int, device, train_ratio: float | None = None):
        spec = WORKLOADS[name]
        if spec["kind"] != "rmat":
            raise ValueError("device-side generation is implemented for the R-MAT workloads")
        dev = torch.device(device)
        self.name, self.seed, self.device = name, seed, dev
        self.indptr, self.indices = rmat_csr_device(spec["scale"], spec["edge_factor"], spec["a"], spec["b"],
                                                    spec["c"], seed, dev)
        self.num_nodes = self.indptr.numel() - 1
        self.num_edges = self.indices.numel()
        self.avg_degree = self.num_edges / self.num_nodes
        self.num_features, self.num_classes = spec["dim"], spec["classes"]
        self.num_layers, self.hidden = spec["layers"], spec["hidden"]
        deg = (self.indptr[1:] - self.indptr[:-1]).clamp(min=1).float()
        self.degrees = deg.rsqrt()
        gen = torch.Generator(device=dev).manual_seed(seed + 2)
        ratio = spec["train_ratio"] if train_ratio is None else train_ratio
        self.train_mask = torch.rand(self.num_nodes, device=dev, generator=gen) < ratio
