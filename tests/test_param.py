"""Knob rules and property bags (EPPGCN/param.py)."""
import types

import pytest

from eppgcn_b200.param import backInputProperty, getBlockSize, inputProperty, maskInputProperty


@pytest.mark.parametrize("dim,shape", [(1, (2, 32)), (7, (2, 32)), (8, (4, 16)), (16, (4, 16)), (22, (4, 16)),
                                       (31, (4, 16)), (32, (8, 8)), (64, (8, 8)), (95, (8, 8)), (96, (16, 4)),
                                       (128, (16, 4)), (191, (16, 4)), (192, (32, 2)), (511, (32, 2)),
                                       (512, (32, 2)), (4096, (32, 2))])
def test_block_size_table(dim, shape):                      # EPPGCN/param.py:6-24
    assert getBlockSize(dim) == shape


def _ds(nodes, edges, feats):
    return types.SimpleNamespace(num_nodes=nodes, avg_degree=edges / nodes, avg_edgeSpan=1.0, num_features=feats)


def test_decider_rules():                                   # EPPGCN/param.py:73-127
    p = inputProperty(None, None, None, 32, 32, 8, 100, hiddenDim=16, dataset_obj=_ds(2097152, 35651584, 128))
    p.decider()
    assert p.partSize == 17                                 # int(E/N), whatever --partSize said
    assert p.warpPerBlock_input == min(int(min(8 * (68 + 512 + 400) / 1e3, 40.0) * 1e3 / (68 + 512)), 8)
    assert p.warpPerBlock_hidden == 8
    assert (p.dimWorker_input, p.dimWorker_hidden) == (32, 16)
    assert p.set_input().dimWorker == 32 and p.state_set_input
    assert p.set_hidden().dimWorker == 16 and not p.state_set_input


def test_decider_never_returns_zero_group_size():
    p = inputProperty(sharedMem=100, hiddenDim=16, dataset_obj=_ds(100, 40, 8))
    p.decider()
    assert p.partSize == 1


def test_dataset_is_required():
    with pytest.raises(ValueError):
        inputProperty()


def test_bags():
    m = maskInputProperty("s", "n", "e", "d", 2, 1, 22)
    assert (m.blockx, m.blocky, m.num_layers, m.layer) == (4, 16, 2, 1)
    b = backInputProperty(degrees="deg", dim=128, layer=2)
    assert (b.blockx, b.blocky, b.id, b.numParts) == (16, 4, None, None)
    b.fillProperty(1, 2, 3, 32, 99)
    assert (b.id, b.partPointer, b.edgeList, b.partSize, b.numParts) == (1, 2, 3, 32, 99)
