"""Run under the bounds-checking build of the library (EPPGCN_B200_DEBUG_BOUNDS=1) by
tests/test_gpu_tiles.py in a child process: small aggregations must leave the record empty, and a
plan whose ids lie beyond the declared limits must be reported -- and skipped, not dereferenced."""
import sys

import numpy as np
import torch

from eppgcn_b200 import capi
from oracle import epp_oracle as O
from tests.helpers import assert_close, degrees_of, random_csr, t


def main():
    cuda = torch.device("cuda:0")
    assert capi.DEBUG_BOUNDS and capi.debug_status()[0] == 0, "not the bounds-checking build"
    for kw, dim in ((dict(n=9, avg_deg=2.0, seed=1, empty_frac=0.3), 16), (dict(n=700, avg_deg=6.0, seed=3, hubs=3, hub_deg=650), 22),
                    (dict(n=128, avg_deg=40.0, seed=4), 64)):
        indptr, indices = random_csr(**kw)
        n = len(indptr) - 1
        deg = degrees_of(indptr)
        feat = np.random.Generator(np.random.PCG64(dim)).standard_normal((n, dim)).astype(np.float32)
        plan = capi.TilePlan.from_csr(t(indptr, cuda), t(indices, cuda))
        src = torch.zeros(n, (dim + 7) // 8 * 8, device=cuda)[:, :dim]
        src.copy_(t(feat * deg[:, None], cuda))
        got = capi.spmm_tiles(src, plan, t(deg, cuda))
        assert_close(got.cpu().numpy(), O.spmm_forward(indptr, indices, deg, feat), 2e-5, 2e-6, what=f"dim {dim}")
        assert capi.debug_status() == (0, 0, 0, 0)
    # source ids beyond the declared source count: the source matrix really has only `half` rows
    indptr, indices = random_csr(n=200, avg_deg=5.0, seed=5)
    n, half = len(indptr) - 1, 100
    assert indices.max() >= half
    plan = capi.TilePlan.from_csr(t(indptr, cuda), t(indices, cuda), num_sources=half)
    src = torch.ones(half, 16, device=cuda)
    out = capi.spmm_tiles(src, plan)
    code, value, limit, _ = capi.debug_status()
    assert code == 1 and value >= half and limit == half, (code, value, limit)
    counts = np.array([(indices[indptr[r]:indptr[r + 1]] < half).sum() for r in range(n)], dtype=np.float32)
    assert np.array_equal(out.cpu().numpy()[:, 0], counts), "ids in range must still be summed, the others skipped"
    assert capi.debug_status() == (0, 0, 0, 0), "reading the record clears it"
    print("bounds cases ok")


if __name__ == "__main__":
    sys.exit(main())
