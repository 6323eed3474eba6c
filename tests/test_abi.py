"""The C-ABI library on a machine without a GPU: it loads, exports exactly what
the header declares, its host entry points match the oracle, and device entry
points refuse bad arguments before touching CUDA."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from eppgcn_b200 import capi
from oracle import epp_oracle as O
from tests.helpers import random_csr

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "eppgcn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(eppgcn_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = header_symbols()
    assert len(names) >= 20
    handle = ctypes.CDLL(capi.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in the header but not exported"
    assert sorted(capi.SIGNATURES) == names, "capi.SIGNATURES and the header disagree"


def test_version_and_status_strings():
    l = capi.lib()
    assert l.eppgcn_version() >= 100
    assert l.eppgcn_status_string(0) == b"EPP_OK"
    assert l.eppgcn_status_string(3) == b"EPP_ERR_SCAN_TIMEOUT"


@settings(max_examples=40, deadline=None)
@given(n=st.integers(1, 60), avg=st.floats(0.0, 7.0), seed=st.integers(0, 10_000), ps=st.integers(1, 9),
       empty=st.sampled_from([0.0, 0.4]))
def test_build_part_host_matches_oracle(n, avg, seed, ps, empty):
    indptr, _ = random_csr(n, avg, seed, empty_frac=empty)
    pp, p2n = capi.build_part(ps, torch.from_numpy(indptr))
    want = O.build_part(ps, indptr)
    assert pp.dtype == torch.int32 and np.array_equal(pp.numpy(), want[0])
    assert np.array_equal(p2n.numpy(), want[1])


def test_build_part_rejects_bad_part_size():
    with pytest.raises(capi.EppError) as e:
        capi.build_part(0, torch.tensor([0, 1], dtype=torch.int32))
    assert e.value.status == capi.EPP_ERR_BAD_ARG


def test_part_size_rules_match_oracle():
    for nodes, length in [(3, 17), (1000, 10000), (1_900_000, 28_000_000), (47, 470_000)]:
        deg = np.zeros(nodes + 5, dtype=np.int32)
        deg[:nodes] = 1
        assert capi.map_back_part_size(nodes, length) == O.get_map_back_part_size(deg, length)
        assert capi.bucket_back_part_size(nodes, length) == O.bucket_back_part_size(length, nodes)
    # C round() is half away from zero
    assert capi.map_back_part_size(1, 0) == 1      # 0.65538 + tiny -> 1


def test_ginfo_host_matches_oracle():
    rng = np.random.Generator(np.random.PCG64(5))
    deg = rng.integers(0, 300, 5000).astype(np.int32)
    got = capi.get_ginfo(torch.from_numpy(deg), 123456).numpy()
    np.testing.assert_allclose(got, O.get_ginfo(deg, 123456), rtol=1e-6)


def test_device_entry_points_validate_before_launching():
    l = capi.lib()
    # dim < 1
    assert l.eppgcn_spmm_forward(None, 0, None, 0, None, None, None, None, None, None, 4, 0, 0, 1, 1, 1, None) \
        == capi.EPP_ERR_BAD_ARG
    assert b"dim" in l.eppgcn_last_error()
    # part size < 1
    assert l.eppgcn_split_parts(None, 4, 0, None, 0, None, 0, None, None, 0, None) == capi.EPP_ERR_BAD_ARG
    assert l.eppgcn_compact_mask(None, None, None, None, -1, None, 0, None, None, 0, None) == capi.EPP_ERR_BAD_ARG
    assert l.eppgcn_compact_scratch_bytes(0) >= 256 + 8
    assert l.eppgcn_compact_scratch_bytes(4097) == 256 + 16
    assert l.eppgcn_split_scratch_bytes(2048) == 256 + 8


def test_python_layer_refuses_cpu_tensors():
    x = torch.zeros(4, 4)
    i = torch.zeros(5, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="must be a 2-D fp32 CUDA tensor|must be a CUDA tensor"):
        capi.spmm_forward(x, i, i, torch.zeros(4), i, i[:4])


def test_operator_module_matches_reference_surface():
    import eppgcn_b200
    g = eppgcn_b200.load_gnnadvisor()
    for name in ("forward", "backward", "mask_forward", "ours_backward", "print_time", "clear_time",
                 "build_part", "build_back_part", "compact_back_edge", "get_map_back_part_size",
                 "split_back_part", "get_ginfo"):            # EPPGCN.cpp:388-403
        assert callable(getattr(g, name))
    x = torch.zeros(2, 2)
    i = torch.zeros(3, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="input must be a CUDA tensor"):      # EPPGCN.cpp:73,91
        g.forward(x, x, i, i, torch.zeros(2), i, i[:2], 1, 1, 1)
    with pytest.raises(RuntimeError, match="d_output must be a CUDA tensor"):   # EPPGCN.cpp:172
        g.ours_backward(x, x, x, i, i, i, torch.zeros(2), 1, 1, 1, 4, 16)
    with pytest.raises(RuntimeError, match="id must be a CUDA tensor"):         # EPPGCN.cpp:145
        g.mask_forward(i, i, i, x.bool(), x.bool(), i, i, 2, 1, 4, 16)
    pp, p2n = g.build_part(2, torch.tensor([0, 3, 3, 4], dtype=torch.int32))
    assert pp.tolist() == [0, 2, 3, 4] and p2n.tolist() == [0, 0, 2]
    # the caller's conversion (EPPGCN/gcn_main.py:127-128) is a no-op on int32
    assert pp.int().dtype == torch.int32
