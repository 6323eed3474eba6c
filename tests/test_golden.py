"""Pins the CPU oracle to outputs of the reference's own operators stored
under tests/golden/ (made by tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from oracle import epp_oracle as O
from tests.golden import make_golden as G
from tests.helpers import assert_close, random_csr

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    path = os.path.join(HERE, name)
    if not os.path.exists(path):
        pytest.skip(f"{name} has not been generated")
    return np.load(path)


def test_oracle_matches_reference_cpu_operators():
    z = load("ref_cpu_ops.npz")
    for i, c in enumerate(G.CPU_CASES):
        c = dict(c)
        ps = c.pop("ps")
        indptr, _ = random_csr(**c)
        pp, p2n = O.build_part(ps, indptr, reference_quirk=True)
        assert np.array_equal(z[f"build_part_{i}_ptr"].astype(np.int64), pp)
        assert np.array_equal(z[f"build_part_{i}_node"].astype(np.int64), p2n)
        deg = np.diff(indptr).astype(np.int32)
        np.testing.assert_allclose(O.get_ginfo(deg, int(deg.sum())), z[f"ginfo_{i}"], rtol=1e-6)


def oracle_gpu_case():
    g = G.golden_inputs()
    path, ngh = O.prepare_execution_path(g["indptr"], g["indices"], g["train"], G.GPU_LAYERS, G.GPU_PART,
                                         [G.GPU_BACK] * G.GPU_LAYERS)
    return g, path, ngh


def test_oracle_matches_reference_cuda_preparation():
    z = load("ref_gpu_ops.npz")
    g, path, ngh = oracle_gpu_case()
    e = len(g["indices"])
    for i in range(G.GPU_LAYERS - 1):
        assert np.array_equal(z[f"ngh_mask_{i}"], ngh[i])
    for i, conv in enumerate(path):
        assert np.array_equal(z[f"edge_mask_{i}"], conv["edge_mask"])
        assert np.array_equal(z[f"node_degs_{i}"], conv["node_degs"])
        assert int(z[f"valid_len_{i}"]) == conv["valid_len"]
        assert np.array_equal(z[f"compact_id_{i}"], conv["id"])
        assert np.array_equal(z[f"compact_edge_{i}"], conv["edgeList"])
        assert O.split_reference_valid(conv["node_degs"], G.GPU_BACK)
        assert int(z[f"num_parts_{i}"]) == conv["numParts"]
        assert np.array_equal(z[f"part_pointer_{i}"], conv["partPointer"][:e])
        assert int(z[f"map_size_{i}"]) == O.get_map_back_part_size(conv["node_degs"], conv["valid_len"])
        ps = O.bucket_back_part_size(conv["valid_len"], O.count_nonzero(conv["node_degs"]))
        want, nparts = O.split_back_part(conv["node_degs"], e, ps)
        np.testing.assert_array_equal(z[f"bbp_info_{i}"], np.array([ps, nparts], dtype=np.float32))
        assert np.array_equal(z[f"bbp_part_pointer_{i}"], want)


@pytest.mark.parametrize("conv", ["rsqrt", "sqrt"])
def test_oracle_matches_reference_cuda_operators(conv):
    z = load("ref_gpu_ops.npz")
    g, path, _ = oracle_gpu_case()
    deg = g[f"deg_{conv}"]
    # the sqrt convention multiplies by degrees instead of normalising, so magnitudes grow with
    # degree; the reference accumulates in fp32 with emulated atomics -> compare relatively
    rtol, atol = (1e-5, 1e-6) if conv == "rsqrt" else (2e-5, 1e-3)
    h = g["x"].astype(np.float64)
    for i in range(G.GPU_LAYERS):
        w = g["ws"][i]
        y = O.gcn_layer_forward(h, w, g["indptr"], g["indices"], deg)
        assert_close(z[f"forward_{conv}_{i}"], y, rtol=10 * rtol, atol=10 * atol, what=f"forward {i}")
        p = path[i]
        d_in, d_w, _ = O.gcn_layer_backward(g["d_outs"][i], h, w, p["id"], p["partPointer"], p["edgeList"], deg,
                                            p["numParts"])
        scale = max(1.0, float(np.abs(d_w).max()))
        assert_close(z[f"ours_backward_{conv}_{i}_dinput"], d_in, rtol=10 * rtol, atol=10 * atol, what="d_input")
        assert_close(z[f"ours_backward_{conv}_{i}_dweight"] / scale, d_w / scale, rtol=1e-4, atol=1e-5,
                     what="d_weight")
        full = O.spmm_forward(g["indptr"], g["indices"], deg, g["d_outs"][i]) @ w.astype(np.float64).T
        assert_close(z[f"backward_{conv}_{i}_dinput"], full, rtol=10 * rtol, atol=10 * atol, what="backward")
        h = np.maximum(z[f"forward_{conv}_{i}"].astype(np.float64), 0)     # follow the reference's activations
