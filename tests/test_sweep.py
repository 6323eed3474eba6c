"""The sweep composes the same flags as the reference's sweep script
(EPPGCN/bench_EPPGCN.py:38-63), and the training CLI parses every one of them."""
import pytest

from eppgcn_b200 import sweep


def test_loop_order_and_mode_mapping():
    runs = sweep.command_lines("regression_equation", "/data")
    assert len(runs) == len(sweep.DATASETS) * len(sweep.RATIOS) * len(sweep.LAYERS)
    first = dict(zip(runs[0][::2], runs[0][1::2]))
    assert first["--dataset"] == "cora" and first["--dim"] == "1433" and first["--classes"] == "7"
    assert first["--train_ratio"] == "0.1" and first["--layers"] == "3" and first["--hidden"] == "16"
    assert first["--backsize_mode"] == "map" and first["--backsize"] == "0" and first["--partSize"] == "0"
    assert first["--dataDir"] == "/data/cora" and first["--loadFromTxt"] == "True"
    second = dict(zip(runs[1][::2], runs[1][1::2]))
    assert second["--layers"] == "4" and second["--train_ratio"] == "0.1"          # layers is the innermost loop
    fixed = sweep.command_lines("fixed_value", "/data", datasets=["pubmed"], ratios=[0.5], layers=[3])
    only = dict(zip(fixed[0][::2], fixed[0][1::2]))
    assert len(fixed) == 1 and only["--backsize_mode"] == "constant" and only["--backsize"] == "32"
    with pytest.raises(SystemExit):
        sweep.command_lines("SAGPG", "/data")
    with pytest.raises(SystemExit):
        sweep.command_lines("fixed_value", "/data", datasets=["nope"])
    with pytest.raises(SystemExit):
        sweep.command_lines("fixed_value", None)


def test_the_training_cli_parses_every_sweep_line():
    from eppgcn_b200 import train
    parser = train.build_parser()
    for argv in sweep.command_lines("regression_equation", "/data") + sweep.command_lines("fixed_value", None,
                                                                                           synthetic=True):
        a = parser.parse_args(argv)
        assert a.model == "gcn" and a.backsize_mode in ("map", "constant")
    a = parser.parse_args(["--dataset", "amazon0601", "--dataDir", "/g", "--backsize_mode", "net"])
    assert a.backsize_mode == "net" and a.loadFromTxt == "True"       # parsed; main() refuses it with a reason
