"""Training harness for the GCN hot path: the call order of the reference's
training script (EPPGCN/gcn_main.py:86-292) as a reusable class plus a CLI
with the same flags and the same printed timing keys.

Sequence (numbers are lines of EPPGCN/gcn_main.py):
  decider (:97) -> build_part (:120) -> CSR and groups to the device (:125-128)
  -> per layer maskInputProperty / backInputProperty (:130-145)
  -> execution-path preparation: one mask_forward per layer, then
     compact_back_edge + part-size rule + split_back_part per layer (:148-168)
  -> Net of GCNConv layers with ReLU between them (:183-208), Adam lr 0.01 (:214)
  -> train(): forward, log_softmax + nll_loss on the train rows, backward,
     optimizer step (:225-265).

The ``net`` part-size mode of the reference needs a PyG predictor with trained
weights that are not part of it; ``map`` (regression rule, clamped to >= 1),
``constant`` and ``bucket`` (the rule inside build_back_part) are provided.
"""
from __future__ import annotations

import argparse
import time

import torch
import torch.nn.functional as F

from . import load_gnnadvisor
from .gcn_conv import GCNConv
from .graphs import WORKLOADS, load_workload
from .param import backInputProperty, inputProperty, maskInputProperty

GNNA = load_gnnadvisor()


class Net(torch.nn.Module):
    """``num_layers`` GCNConv layers, ReLU after all but the last
    (EPPGCN/gcn_main.py:183-208)."""

    def __init__(self, num_layers, in_dim, hidden, num_classes):
        super().__init__()
        self.num_layers = num_layers
        dims = [in_dim] + [hidden] * (num_layers - 1) + [num_classes]
        self.convs = torch.nn.ModuleList(GCNConv(dims[i], dims[i + 1]) for i in range(num_layers))

    def print_time(self):
        self.convs[0].print_time()

    def clear_time(self):
        self.convs[0].clear_time()

    def forward(self, x, inputInfo, mask_props, back_props, isFirstIter, isBackModeNet):
        for i, conv in enumerate(self.convs):
            info = inputInfo.set_input() if i == 0 else inputInfo.set_hidden()
            x = conv(x, info, mask_props[i], back_props[i], isFirstIter, isBackModeNet)
            if i < self.num_layers - 1:
                x = F.relu(x)
        return x


class GCNTrainer:
    """Owns the bags, the prepared execution path, the model and the optimizer."""

    def __init__(self, dataset, hidden=16, backsize_mode="constant", backsize=32,
                 partSize=32, dimWorker=32, warpPerBlock=8, sharedMem=100,
                 prepare_before_training=True, seed=0, device="cuda", manual_mode=False, verbose=False,
                 path_cache_dir=None):
        self.ds = dataset
        self.device = torch.device(device)
        self.layers = dataset.num_layers
        self.hidden = hidden
        self.backsize_mode, self.backsize = backsize_mode, backsize
        self.build_time = 0.0
        ds = dataset
        ds.to(self.device)      # degrees, features and masks live on the GPU; the CSR stays on the host for build_part

        info = inputProperty(ds.row_pointers, ds.column_index, ds.degrees, partSize, dimWorker, warpPerBlock,
                             sharedMem, hiddenDim=hidden, dataset_obj=ds, manual_mode=manual_mode,
                             verbose=verbose)
        info.decider()
        t0 = time.perf_counter()
        partPtr, part2Node = GNNA.build_part(info.partSize, ds.row_pointers.cpu())
        self.build_part_time = time.perf_counter() - t0
        info.row_pointers = ds.row_pointers.to(self.device)
        info.column_index = ds.column_index.to(self.device)
        info.partPtr = partPtr.int().to(self.device)
        info.part2Node = part2Node.int().to(self.device)
        self.inputInfo = info

        L = self.layers
        dims = [hidden] * (L - 1) + [ds.num_classes]
        self.mask_props, self.back_props = [], []
        for i in range(L):
            src = ds.train_mask if i == 0 else ds.ngh_masks[i - 1]
            dst = ds.ngh_masks[i] if i < L - 1 else ds.empty_mask
            self.mask_props.append(maskInputProperty(src, dst, ds.edge_masks[L - 1 - i], ds.node_degs[L - 1 - i],
                                                     L, i + 1, dims[i]))
            self.back_props.append(backInputProperty(degrees=ds.degrees, dim=dims[i], layer=i + 1))

        torch.manual_seed(seed)
        self.model = Net(L, ds.num_features, hidden, ds.num_classes).to(self.device)
        self.optimizer = torch.optim.Adam(self.model.parameters(), lr=0.01)
        self.prepared = self.path_from_cache = False
        self.is_net_order = prepare_before_training
        self.path_cache_dir, self._path_fp = path_cache_dir, None
        if path_cache_dir:
            # a path prepared by an earlier run for the same graph, mask and knobs is read back instead
            from . import path_cache
            t0 = time.perf_counter()
            self._path_fp = path_cache.fingerprint(ds.row_pointers, ds.column_index, ds.train_mask, L, info.partSize,
                                                   backsize_mode, backsize)
            cached = path_cache.load(path_cache_dir, self._path_fp, self.device)
            if cached is not None and len(cached) == L:
                for prop, c in zip(self.back_props, cached):
                    prop.fillProperty(c["id"], c["partPointer"], c["edgeList"], c["partSize"], c["numParts"])
                    prop.valid_len = c["valid_len"]
                self.prepared = self.path_from_cache = True
                self.build_time += time.perf_counter() - t0
        if prepare_before_training and not self.prepared:
            t0 = time.perf_counter()
            for i in range(L):
                self.mask_forward(i)
            self.build_back_part()
            self._sync()
            self.build_time += time.perf_counter() - t0
        self.for_time = self.loss_time = self.back_time = 0.0

    def _sync(self):
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    # EPPGCN/gcn_main.py:147-149
    def mask_forward(self, i):
        m, info = self.mask_props[i], self.inputInfo
        GNNA.mask_forward(info.part2Node, info.partPtr, info.column_index, m.src_mask, m.ngh_mask,
                          m.backEdgeMask, m.node_degs, m.num_layers, m.layer, m.blockx, m.blocky)

    def choose_back_size(self, i, valid_len):
        if self.backsize_mode == "map":
            return max(GNNA.get_map_back_part_size(self.ds.node_degs[i], valid_len), 1)
        if self.backsize_mode == "bucket":
            nodes = int(torch.count_nonzero(self.ds.node_degs[i]).item())
            d = valid_len // max(nodes, 1)
            return 4 if d < 4 else 8 if d < 16 else 16 if d < 64 else 32 if d < 256 else 64
        if self.backsize_mode == "constant":
            return max(int(self.backsize), 1)
        raise ValueError("backsize_mode must be map, bucket or constant")

    # EPPGCN/gcn_main.py:151-168
    def build_back_part(self):
        ds = self.ds
        for i in range(self.layers):
            ids, edge_list, valid = GNNA.compact_back_edge(ds.edge_masks[i], self.inputInfo.column_index)
            valid_len = int(valid[0].item())
            ps = self.choose_back_size(i, valid_len)
            part_pointer, nparts = GNNA.split_back_part(ds.node_degs[i], ds.num_edges, ps)
            self.back_props[i].fillProperty(ids, part_pointer, edge_list, ps, int(nparts[0].item()))
            self.back_props[i].valid_len = valid_len
        self.prepared = True
        if self.path_cache_dir:
            from . import path_cache
            path_cache.save(self.path_cache_dir, self._path_fp, self.back_props)

    def forward(self, x=None, isFirstIter=False):
        return self.model(self.ds.x if x is None else x, self.inputInfo, self.mask_props, self.back_props,
                          isFirstIter, self.is_net_order)

    # EPPGCN/gcn_main.py:225-265
    def train_epoch(self, isFirstIter=False, timed=False, x=None):
        if self.path_from_cache:
            isFirstIter = False                      # nothing to mark or to build: the path came from disk
        self.model.train()
        self.optimizer.zero_grad()
        t0 = time.perf_counter()
        out = self.forward(x, isFirstIter)
        if timed:
            self._sync()
            self.for_time += time.perf_counter() - t0
        if isFirstIter and not self.prepared:
            t0 = time.perf_counter()
            self.build_back_part()
            self.build_time += time.perf_counter() - t0
        t0 = time.perf_counter()
        logp = F.log_softmax(out, dim=1)
        loss = F.nll_loss(logp[self.ds.train_mask], self.ds.y[self.ds.train_mask])
        if timed:
            self._sync()
            self.loss_time += time.perf_counter() - t0
        t0 = time.perf_counter()
        loss.backward()
        if timed:
            self._sync()
            self.back_time += time.perf_counter() - t0
        self.optimizer.step()
        return loss


def build_parser() -> argparse.ArgumentParser:
    """The flags of the reference's training script (EPPGCN/gcn_main.py:19-52),
    so that its sweep script's command lines parse unchanged."""
    p = argparse.ArgumentParser(description="GCN training on a seeded synthetic workload, or on the reference's "
                                            "graph files when --dataDir is given")
    p.add_argument("--dataDir", default=None,
                   help="folder with <dataset>_snap or <dataset>.npz and train_mask_<ratio> (EPPGCN/gcn_main.py:21,73-78)")
    p.add_argument("--loadFromTxt", default="True", choices=["True", "False"])
    p.add_argument("--dataset", default="pubmed",
                   help="a synthetic workload (" + ", ".join(sorted(WORKLOADS)) + ") or, with --dataDir, a file stem")
    p.add_argument("--dim", type=int, default=None)
    p.add_argument("--hidden", type=int, default=None)
    p.add_argument("--classes", type=int, default=None)
    p.add_argument("--layers", type=int, default=None)
    p.add_argument("--train_ratio", type=float, default=None)
    p.add_argument("--num_epoches", type=int, default=100)
    p.add_argument("--partSize", type=int, default=32)
    p.add_argument("--dimWorker", type=int, default=32)
    p.add_argument("--warpPerBlock", type=int, default=8)
    p.add_argument("--sharedMem", type=int, default=100)
    p.add_argument("--backsize", type=int, default=32)
    p.add_argument("--backsize_mode", default="constant", choices=["map", "net", "bucket", "constant"])
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--path_cache", default=None,
                   help="folder for prepared execution paths; a matching one is loaded instead of prepared again")
    p.add_argument("--model", default="gcn", choices=["gcn", "gin"])
    for flag in ("--manual_mode", "--verbose_mode", "--single_spmm", "--verify_spmm"):
        p.add_argument(flag, default="False", choices=["True", "False"])
    return p


def main(argv=None):
    a = build_parser().parse_args(argv)
    if a.model != "gcn":
        raise SystemExit("only the GCN path is built (the GIN layers of the reference's script are commented out)")
    if a.backsize_mode == "net":
        raise SystemExit("--backsize_mode net needs the reference's trained PyG part-size predictor, which is not "
                         "part of it; use map, bucket or constant")
    if a.single_spmm == "True" or a.verify_spmm == "True":
        raise SystemExit("--single_spmm / --verify_spmm: use bench.py --kernels-only and the parity tests instead")
    if not torch.cuda.is_available():
        raise SystemExit("a CUDA device is required (there is no CPU fallback)")
    if a.dataDir is not None:
        # the reference's defaults (EPPGCN/gcn_main.py:23-27)
        spec = dict(hidden=16, train_ratio=0.1)
        from .loader import load_dataset_files
        ds = load_dataset_files(a.dataDir, a.dataset, a.train_ratio if a.train_ratio is not None else 0.1,
                                a.dim or 96, a.classes or 22, a.layers or 2,
                                load_from_txt=a.loadFromTxt == "True", seed=a.seed)
    else:
        if a.dataset not in WORKLOADS:
            raise SystemExit(f"unknown workload {a.dataset!r}; give --dataDir to read graph files")
        spec = WORKLOADS[a.dataset]
        ds = load_workload(a.dataset, a.seed, train_ratio=a.train_ratio, layers=a.layers)
        if a.dim is not None or a.classes is not None:
            raise SystemExit("--dim/--classes are fixed by the synthetic workloads")
    ratio = a.train_ratio if a.train_ratio is not None else spec["train_ratio"]
    print("||{}   {}   {}".format(a.dataset, ratio, ds.num_layers))
    tr = GCNTrainer(ds, hidden=a.hidden or spec["hidden"], backsize_mode=a.backsize_mode, backsize=a.backsize,
                    partSize=a.partSize, dimWorker=a.dimWorker, warpPerBlock=a.warpPerBlock,
                    sharedMem=a.sharedMem, prepare_before_training=False, seed=a.seed,
                    manual_mode=a.manual_mode == "True", verbose=a.verbose_mode == "True",
                    path_cache_dir=a.path_cache)
    for i in range(10):                       # dry run, EPPGCN/gcn_main.py:272-273
        tr.train_epoch(i == 0, timed=True)
    tr.for_time = tr.loss_time = tr.back_time = 0.0
    tr.model.clear_time()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(a.num_epoches):
        tr.train_epoch(False, timed=True)
    torch.cuda.synchronize()
    total = time.perf_counter() - t0
    tr.model.print_time()
    print("for_time: {:.6f}".format(tr.for_time))
    print("loss_time: {:.6f}".format(tr.loss_time))
    print("back_time: {:.6f}".format(tr.back_time))
    print("build_time: {:.6f}".format(tr.build_time))
    print("Time: {:.6f}".format(total))
    print()


if __name__ == "__main__":
    main()
