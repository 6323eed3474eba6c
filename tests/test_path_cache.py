"""Round trip of a prepared execution path through the on-disk cache, and the
cases in which a file must not be used."""
import types

import numpy as np
import torch

from eppgcn_b200 import path_cache
from oracle import epp_oracle as O
from tests.helpers import random_csr


def _props(indptr, indices, train, layers, sizes):
    path, _ = O.prepare_execution_path(indptr, indices, train, layers, 4, sizes)
    props = []
    for conv in path:
        e = len(indices)
        ids = np.zeros(e, np.int32); ids[:conv["valid_len"]] = conv["id"][:conv["valid_len"]]
        edges = np.zeros(e, np.int32); edges[:conv["valid_len"]] = conv["edgeList"][:conv["valid_len"]]
        ptr = np.zeros(e + 1, np.int32); ptr[:conv["numParts"] + 1] = conv["partPointer"][:conv["numParts"] + 1]
        props.append(types.SimpleNamespace(id=torch.from_numpy(ids), edgeList=torch.from_numpy(edges),
                                           partPointer=torch.from_numpy(ptr), partSize=conv["partSize"],
                                           numParts=conv["numParts"], valid_len=conv["valid_len"]))
    return props


def test_round_trip_and_rejections(tmp_path):
    indptr, indices = random_csr(n=300, avg_deg=4.0, seed=2)
    train = np.random.Generator(np.random.PCG64(1)).random(300) < 0.2
    props = _props(indptr, indices, train, 2, [8, 8])
    args = (torch.from_numpy(indptr), torch.from_numpy(indices), torch.from_numpy(train), 2, 4, "constant", 8)
    fp = path_cache.fingerprint(*args)
    assert path_cache.load(str(tmp_path), fp) is None                       # nothing there yet
    file = path_cache.save(str(tmp_path), fp, props)
    got = path_cache.load(str(tmp_path), fp)
    assert got is not None and len(got) == 2
    for g, p in zip(got, props):
        assert g["numParts"] == p.numParts and g["valid_len"] == p.valid_len and g["partSize"] == p.partSize
        assert torch.equal(g["id"], p.id[:p.valid_len]) and torch.equal(g["edgeList"], p.edgeList[:p.valid_len])
        assert torch.equal(g["partPointer"], p.partPointer[:p.numParts + 1])
        assert g["id"].dtype == torch.int32 and g["partPointer"].dtype == torch.int32
    # any input of the preparation changes the fingerprint
    other_mask = train.copy(); other_mask[0] = not other_mask[0]
    variants = [(args[0], args[1], torch.from_numpy(other_mask), 2, 4, "constant", 8),
                (args[0], args[1], args[2], 3, 4, "constant", 8),
                (args[0], args[1], args[2], 2, 5, "constant", 8),
                (args[0], args[1], args[2], 2, 4, "map", 8),
                (args[0], args[1], args[2], 2, 4, "constant", 16)]
    assert len({path_cache.fingerprint(*v) for v in variants} | {fp}) == len(variants) + 1
    assert all(path_cache.load(str(tmp_path), path_cache.fingerprint(*v)) is None for v in variants)
    # a damaged file is ignored, not trusted
    with open(file, "r+b") as f:
        f.truncate(100)
    assert path_cache.load(str(tmp_path), fp) is None
