"""The reference's experiment sweep (EPPGCN/bench_EPPGCN.py) without its
absolute paths: every dataset x train ratio x layer count runs the training
harness once with the flags that script composes (EPPGCN/bench_EPPGCN.py:55-61).

``--groupsize_model`` keeps the reference's three names:
``regression_equation`` -> ``--backsize_mode map``, ``fixed_value`` ->
``--backsize_mode constant --backsize 32``; ``SAGPG`` (the PyG predictor with
trained weights) is not part of the reference's repository and is refused.

    python -m eppgcn_b200.sweep --dataRoot /data/graphs --datasets cora pubmed
    python -m eppgcn_b200.sweep --synthetic                # the seeded stand-ins

``--backsize-sweep`` is the brute-force search of EPPGCN/best_partSize_test.sh:35-60,76-86 (every
backward part size, best by ``l{k}_back_agg_time``) done in one process on the device: the path is
prepared once, every size only repeats the part splitting and times each layer's compacted backward
aggregation with CUDA events.  It times the group kernel, whose work units are the parts; the planned
tile kernel the operator module uses by default builds its units from the compacted row ids and does not
depend on the part size -- its time is printed beside the sweep for comparison.

    python -m eppgcn_b200.sweep --backsize-sweep 1 2 4 8 16 32 64 --workload rmat21
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


def backsize_sweep(workload: str, sizes, train_ratio=None, seed: int = 0, reps: int = 10, device="cuda"):
    """Times every layer's compacted backward aggregation for every part size in ``sizes``.
    Returns ``{"layers": [{"dim", "active_edges", "ms": {size: ms}, "best", "tiles_ms"}, ...]}``."""
    import torch
    import eppgcn_b200
    from . import capi, graphs
    dev = torch.device(device)
    gnna = eppgcn_b200.load_gnnadvisor()
    spec = graphs.WORKLOADS[workload]
    ds = graphs.load_workload(workload, seed, train_ratio=train_ratio)
    n, e, L = ds.num_nodes, ds.num_edges, ds.num_layers
    part = max(int(ds.avg_degree), 1)
    pp, p2n = gnna.build_part(part, ds.row_pointers)
    col, pp, p2n, deg = ds.column_index.to(dev), pp.to(dev), p2n.to(dev), ds.degrees.to(dev)
    ds.to(dev)
    for i in range(L):
        src = ds.train_mask if i == 0 else ds.ngh_masks[i - 1]
        dst = ds.ngh_masks[i] if i < L - 1 else ds.empty_mask
        gnna.mask_forward(p2n, pp, col, src, dst, ds.edge_masks[L - 1 - i], ds.node_degs[L - 1 - i], L, i + 1, 4, 16)
    dims = [spec["hidden"]] * (L - 1) + [spec["classes"]]
    gen = torch.Generator(device=dev).manual_seed(seed)

    def timed(fn):
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b) / reps

    layers = []
    for i in range(L):
        ids, edges, info = gnna.compact_back_edge(ds.edge_masks[i], col)
        valid = int(info[0].item())
        d_out = torch.randn(n, dims[i], device=dev, generator=gen)
        out = torch.empty(n, dims[i], device=dev)
        ms = {}
        for ps in sizes:
            ppb, pinfo = gnna.split_back_part(ds.node_degs[i], e, int(ps))
            parts = int(pinfo[0].item())
            ms[int(ps)] = round(timed(lambda: capi.spmm_backward_compacted(d_out, ids, ppb, edges, deg, parts, int(ps),
                                                                        out=out)), 4)
        plan = capi.TilePlan.from_ids(ids, edges, valid, n)
        src = capi.pack_scaled_rows(d_out, deg, plan)
        tiles = timed(lambda: (capi.pack_scaled_rows(d_out, deg, plan, out=src), capi.spmm_tiles(src, plan, deg, out=out)))
        layers.append({"layer": i + 1, "dim": dims[i], "active_edges": valid, "ms": ms,
                       "best": min(ms, key=ms.get), "tiles_ms": round(tiles, 4)})
    return {"workload": workload, "train_ratio": spec["train_ratio"] if train_ratio is None else train_ratio,
            "layers": layers}


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
    p.add_argument("--backsize-sweep", nargs="+", type=int, default=None, metavar="SIZE",
                   help="time every layer's compacted backward aggregation for these part sizes on the device")
    p.add_argument("--workload", default="rmat21", help="--backsize-sweep: the synthetic workload")
    p.add_argument("--train_ratio", type=float, default=None, help="--backsize-sweep: train mask ratio")
    a = p.parse_args(argv)
    if a.backsize_sweep:
        import json
        res = backsize_sweep(a.workload, a.backsize_sweep, a.train_ratio)
        for lay in res["layers"]:
            print(f"l{lay['layer']}_back_agg_time (ms) by part size, dim {lay['dim']}, {lay['active_edges']} active edges: "
                  + ", ".join(f"{k}: {v}" for k, v in lay["ms"].items())
                  + f"  -> best {lay['best']}; planned tile kernel (any size): {lay['tiles_ms']}")
        print(json.dumps(res))
        return
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
