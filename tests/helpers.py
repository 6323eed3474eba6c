"""Small seeded inputs shared by the CPU and GPU tests."""
import numpy as np
import torch

from oracle import epp_oracle as O


def random_csr(n, avg_deg, seed, empty_frac=0.0, hubs=0, hub_deg=0, self_loops=False):
    """Random CSR with sorted, distinct columns; optional empty rows and hubs."""
    rng = np.random.Generator(np.random.PCG64(seed))
    deg = rng.poisson(avg_deg, n).astype(np.int64)
    deg = np.minimum(deg, n)
    if empty_frac:
        deg[rng.random(n) < empty_frac] = 0
    for h in rng.choice(n, size=min(hubs, n), replace=False):
        deg[h] = min(hub_deg, n)
    cols = []
    for r in range(n):
        c = rng.choice(n, size=int(deg[r]), replace=False)
        if self_loops and deg[r] and r not in c:
            c[0] = r
        cols.append(np.sort(c))
    indptr = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(deg, out=indptr[1:])
    indices = np.concatenate(cols).astype(np.int32) if n and indptr[-1] else np.zeros(0, dtype=np.int32)
    return indptr, indices


def degrees_of(indptr, kind="rsqrt"):
    d = np.maximum(np.diff(indptr), 1).astype(np.float32)
    return (1.0 / np.sqrt(d)).astype(np.float32) if kind == "rsqrt" else np.sqrt(d).astype(np.float32)


def t(a, device, dtype=None):
    x = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        x = x.to(dtype)
    return x.to(device)


def assert_close(got, want, rtol=O.RTOL, atol=O.ATOL, what=""):
    """|got - want| <= atol + rtol*|want| elementwise, against a float64 oracle."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    err = np.abs(got - want) - (atol + rtol * np.abs(want))
    bad = int((err > 0).sum())
    assert bad == 0, f"{what}: {bad} of {got.size} elements off, worst excess {err.max():.3e}"


def prepared_path(indptr, indices, train_mask, layers, part_size, back_sizes):
    """Oracle preparation, returned per convolution."""
    return O.prepare_execution_path(indptr, indices, train_mask, layers, part_size, back_sizes)


def cached_path_scenario(tmp_path, device, make_trainer=None):
    """Two trainers on the same workload and seed: the first prepares the
    execution path and writes it to ``tmp_path``, the second must load it and
    take the same first step.  Shared by the GPU test and by the CPU test that
    runs the harness on a numpy double of the operator module."""
    import pytest
    import torch
    from eppgcn_b200 import graphs
    from eppgcn_b200.train import GCNTrainer

    def run():
        ds = graphs.load_workload("cora", 0)
        tr = GCNTrainer(ds, hidden=16, backsize_mode="map", prepare_before_training=False, seed=5,
                        path_cache_dir=str(tmp_path), device=device)
        losses = [float(tr.train_epoch(i == 0).item()) for i in range(4)]
        return tr, losses

    first, l1 = run()
    assert not first.path_from_cache and first.prepared and len(list(tmp_path.iterdir())) == 1
    second, l2 = run()
    assert second.path_from_cache and second.prepared
    for a, b in zip(first.back_props, second.back_props):
        assert a.numParts == b.numParts and a.partSize == b.partSize and a.valid_len == b.valid_len
        assert torch.equal(a.id[:a.valid_len], b.id) and torch.equal(a.edgeList[:a.valid_len], b.edgeList)
        assert torch.equal(a.partPointer[:a.numParts + 1], b.partPointer)
    # the first step starts from the same weights (atomics may reorder sums); later ones only have to stay sane
    assert l1[0] == pytest.approx(l2[0], rel=1e-5) and all(np.isfinite(l1 + l2))
    return first, second
