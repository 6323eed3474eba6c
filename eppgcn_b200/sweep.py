"""The reference's experiment sweep (EPPGCN/bench_EPPGCN.py) without its
absolute paths: every dataset x train ratio x layer count runs the training
harness once with the flags that script composes (EPPGCN/bench_EPPGCN.py:55-61).

``--groupsize_model`` keeps the reference's three names:
``regression_equation`` -> ``--backsize_mode map``, ``fixed_value`` ->
``--backsize_mode constant --backsize 32``; ``SAGPG`` (the PyG predictor with
trained weights) is not part of the reference's repository and is refused.

    python -m eppgcn_b200.sweep --dataRoot /data/graphs --datasets cora pubmed
    python -m eppgcn_b200.sweep --synthetic                # the seeded stand-ins
"""
from __future__ import annotations

import argparse

# name, input dimension, classes (EPPGCN/bench_EPPGCN.py:17-30)
DATASETS = [("cora", 1433, 7), ("citeseer", 3703, 6), ("pubmed", 500, 3), ("youtube", 64, 47), ("amazon", 96, 22),
            ("corafull", 64, 32), ("catalog", 64, 32), ("twitter", 64, 32), ("google", 64, 32), ("dblp", 64, 32)]
RATIOS = [0.1, 0.3, 0.5, 0.8]            # EPPGCN/bench_EPPGCN.py:32
LAYERS = [3, 4, 5, 6]                    # EPPGCN/bench_EPPGCN.py:36
HIDDEN = [16]                            # EPPGCN/bench_EPPGCN.py:15
SYNTHETIC = ["cora", "pubmed", "social"]


def back_mode(groupsize_model: str):
    """``(backsize_mode, backsize)`` for a sweep mode (EPPGCN/bench_EPPGCN.py:47-53)."""
    if groupsize_model == "regression_equation":
        return "map", 0
    if groupsize_model == "fixed_value":
        return "constant", 32
    if groupsize_model == "SAGPG":
        raise SystemExit("SAGPG needs the trained PyG part-size predictor, which the reference does not ship")
    raise ValueError(f"unknown groupsize_model {groupsize_model!r}")


def command_lines(groupsize_model: str, data_root: str | None, datasets=None, ratios=None, layers=None,
                  synthetic: bool = False, epochs: int | None = None):
    """The argument vectors of one sweep, in the reference's loop order
    (hidden, dataset, ratio, layers)."""
    mode, backsize = back_mode(groupsize_model)
    out = []
    if synthetic:
        table = [(name, None, None) for name in (datasets or SYNTHETIC)]
    else:
        if not data_root:
            raise SystemExit("--dataRoot is required unless --synthetic is given")
        wanted = set(datasets) if datasets else None
        table = [row for row in DATASETS if wanted is None or row[0] in wanted]
        missing = (wanted or set()) - {row[0] for row in table}
        if missing:
            raise SystemExit("unknown dataset(s): " + ", ".join(sorted(missing)))
    for hid in HIDDEN:
        for name, dim, classes in table:
            for ratio in (ratios or RATIOS):
                for layer in (layers or LAYERS):
                    argv = ["--dataset", name, "--hidden", str(hid), "--layers", str(layer), "--partSize", "0",
                            "--model", "gcn", "--warpPerBlock", "8", "--manual_mode", "False",
                            "--verbose_mode", "False", "--train_ratio", str(ratio),
                            "--backsize_mode", mode, "--backsize", str(backsize)]
                    if not synthetic:
                        argv += ["--dim", str(dim), "--classes", str(classes), "--loadFromTxt", "True",
                                 "--dataDir", data_root.rstrip("/") + "/" + name]
                    if epochs is not None:
                        argv += ["--num_epoches", str(epochs)]
                    out.append(argv)
    return out


def main(argv=None):
    p = argparse.ArgumentParser(description="dataset x train ratio x layers sweep of the training harness")
    p.add_argument("--groupsize_model", default="regression_equation",
                   choices=["regression_equation", "SAGPG", "fixed_value"])
    p.add_argument("--dataRoot", default=None, help="folder holding one sub-folder of graph files per dataset")
    p.add_argument("--synthetic", action="store_true", help="sweep the seeded synthetic workloads instead of files")
    p.add_argument("--datasets", nargs="*", default=None)
    p.add_argument("--ratios", nargs="*", type=float, default=None)
    p.add_argument("--layers", nargs="*", type=int, default=None)
    p.add_argument("--num_epoches", type=int, default=None)
    p.add_argument("--dry_run", action="store_true", help="print the command lines only")
    a = p.parse_args(argv)
    runs = command_lines(a.groupsize_model, a.dataRoot, a.datasets, a.ratios, a.layers, a.synthetic, a.num_epoches)
    if a.dry_run:
        for r in runs:
            print("python -m eppgcn_b200.train " + " ".join(r))
        return
    from . import train
    for r in runs:
        train.main(r)


if __name__ == "__main__":
    main()
