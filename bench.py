#!/usr/bin/env python
"""Benchmark of the GCN aggregation hot path.

Metric: ms per epoch of the forward + backward neighbour aggregation of a
2-layer GCN (hidden 16, 22 classes) -- two forward SpMMs over the whole graph
and two backward SpMMs over the prepared execution path -- on a seeded R-MAT
scale-21 graph (2,097,152 vertices, 35,651,584 directed edges with self loops).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

* ``value``  device-resident: inputs already in HBM, K steps timed with CUDA
  events around the C-ABI launches.
* ``e2e``    the same four aggregations through the C-ABI with HOST buffers:
  every step copies its four input matrices from pinned host memory and
  copies the four results back.
* ``roofline``  the dominant kernel's compulsory bytes / its CUDA-event time,
  against the measured HBM copy bandwidth.
* ``cpu_baseline`` / ``--impl reference``  the CPU GCN path (torch.sparse CSR
  SpMM, fp32, all host cores) on the same graph: the same four aggregations,
  over the whole graph in both directions (the CPU path has no execution-path
  preparation).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of each aggregation kernel on the default
# workload (rmat21, seed 0), from the ncu capture summarised in profiles/staged_spmm_rmat21_ncu_full.md.
NCU_DRAM_TRAFFIC = {"fwd_d16": 590_400_000, "fwd_d22": 903_200_000,
                    "bwd_conv2_d22": 136_700_000, "bwd_conv1_d16": 492_700_000}


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def measured_peak_gbs():
    """(GB/s, source) of the HBM roofline denominator."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
            time.sleep(0.6)          # nvidia-smi needs a moment before its first sample
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


_probe_lib = None


def probe_gather(col_idx, feat, sink):
    """Enqueues the bare gather of ``feat`` rows over ``col_idx`` (the benchmark's own measurement
    library, built beside the package; not part of the product's C-ABI)."""
    import ctypes as C
    global _probe_lib
    if _probe_lib is None:
        from eppgcn_b200 import build
        _probe_lib = C.CDLL(build.build_probe())
        _probe_lib.eppgcn_probe_gather.restype = C.c_int
        _probe_lib.eppgcn_probe_gather.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_int,
                                                   C.c_void_p, C.c_void_p]
    rc = _probe_lib.eppgcn_probe_gather(col_idx.data_ptr(), col_idx.numel(), feat.data_ptr(), feat.stride(0),
                                        feat.size(1), sink.data_ptr(), torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"eppgcn_probe_gather failed with status {rc}")


# ---------------------------------------------------------------------------
# CPU GCN path (reference arm and cpu_baseline)
# ---------------------------------------------------------------------------
def run_cpu(graph, dims, steps, warmup, budget_s=25.0):
    """Times the CPU path through the oracle module; returns (ms/epoch, cores, epochs timed)."""
    from oracle import cpu_gcn
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    a = cpu_gcn.normalised_csr(graph)
    g = torch.Generator().manual_seed(0)
    mats = [torch.randn(graph.num_nodes, d, generator=g) for d in (dims[0], dims[1], dims[1], dims[0])]
    for _ in range(max(1, min(warmup, 2))):
        t0 = time.perf_counter()
        cpu_gcn.aggregation_epoch(a, mats)
        one = time.perf_counter() - t0
    epochs = max(1, min(steps, int(budget_s / max(one, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(epochs):
        cpu_gcn.aggregation_epoch(a, mats)
    ms = (time.perf_counter() - t0) * 1e3 / epochs
    return ms, cores, epochs


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class HotPath:
    """Device-resident state of one rank: CSR slice, groups, prepared path."""

    def __init__(self, ds, dev, back_size=32):
        import eppgcn_b200
        from eppgcn_b200 import capi
        self.capi, self.dev = capi, dev
        gnna = eppgcn_b200.load_gnnadvisor()
        n, e, L = ds.num_nodes, ds.num_edges, ds.num_layers
        self.n, self.e = n, e
        self.part_size = max(int(ds.avg_degree), 1)
        t0 = time.perf_counter()
        pp, p2n = gnna.build_part(self.part_size, ds.row_pointers)
        self.build_part_s = time.perf_counter() - t0
        self.row = ds.row_pointers.to(dev); self.col = ds.column_index.to(dev)
        self.pp, self.p2n = pp.to(dev), p2n.to(dev)
        self.deg = ds.degrees.to(dev)
        ds.to(dev)
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for i in range(L):
            src = ds.train_mask if i == 0 else ds.ngh_masks[i - 1]
            dst = ds.ngh_masks[i] if i < L - 1 else ds.empty_mask
            gnna.mask_forward(self.p2n, self.pp, self.col, src, dst, ds.edge_masks[L - 1 - i],
                              ds.node_degs[L - 1 - i], L, i + 1, 4, 16)
        self.path = []
        for i in range(L):
            ids, edges, info = gnna.compact_back_edge(ds.edge_masks[i], self.col)
            ppb, pinfo = gnna.split_back_part(ds.node_degs[i], e, back_size)
            self.path.append(dict(id=ids, edges=edges, pp=ppb, parts=int(pinfo[0].item()),
                                  valid=int(info[0].item()),
                                  rows=int(torch.count_nonzero(ds.node_degs[i]).item())))
        torch.cuda.synchronize(dev)
        self.prep_s = time.perf_counter() - t0
        self.back_size = back_size

    def forward(self, feat, out):
        """Forward aggregation as the operator module runs it: the update step has already folded
        deg[col] into the rows of `feat`."""
        return self.capi.spmm_forward(feat, self.row, self.col, self.deg, self.pp, self.p2n, self.part_size, out=out,
                                      prescaled=True)

    def backward(self, i, d_out, out):
        p = self.path[i]
        return self.capi.spmm_backward_compacted(d_out, p["id"], p["pp"], p["edges"], self.deg, p["parts"],
                                                 self.back_size, out=out)


def padded(n, d, dev, gen):
    """[n, d] view with a row stride that is a multiple of 8 floats, as the forward operator lays out X @ W."""
    ld = (d + 7) // 8 * 8
    full = torch.randn(n, ld, device=dev, generator=gen)
    return full[:, :d]


def bytes_forward(n, e, d):
    return 4 * e + 4 * (n + 1) + 4 * n + 4 * d * n + 4 * d * n


def bytes_backward(n, d, p, src_rows):
    return 4 * p["valid"] + 4 * (p["parts"] + 1) + 4 * p["parts"] + 4 * d * src_rows + 4 * (p["rows"] + src_rows) + 4 * d * n


def run_gpu(args):
    from eppgcn_b200 import graphs
    rank = int(os.environ.get("RANK", 0)); world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    spec0 = graphs.WORKLOADS[args.workload]
    if world > 1 or spec0.get("draw") == "device":
        # several ranks, or a workload that is drawn on the GPU: the row-partitioned driver (also at one rank)
        import bench_multi
        return bench_multi.run_bench(args, rank, world, dev)

    spec = graphs.WORKLOADS[args.workload]
    t0 = time.perf_counter()
    ds = graphs.load_workload(args.workload, args.seed)
    log(f"[bench] workload {args.workload}: N={ds.num_nodes} E={ds.num_edges} ({time.perf_counter() - t0:.1f}s)")
    graph = ds.graph
    n, e = ds.num_nodes, ds.num_edges
    dims = [spec["hidden"], spec["classes"]]
    src_rows = [int(ds.train_mask.sum())]           # rows of d_out the last convolution's backward reads
    hp = HotPath(ds, dev, args.backsize)
    src_rows = [int(ds.ngh_masks[0].sum().item()), int(ds.train_mask.sum().item())]   # conv1, conv2
    gen = torch.Generator(device=dev).manual_seed(args.seed)
    ins = [padded(n, dims[0], dev, gen), padded(n, dims[1], dev, gen),
           torch.randn(n, dims[1], device=dev, generator=gen), torch.randn(n, dims[0], device=dev, generator=gen)]
    outs = [torch.empty(n, d, device=dev) for d in (dims[0], dims[1], dims[1], dims[0])]
    names = [f"fwd_d{dims[0]}", f"fwd_d{dims[1]}", f"bwd_conv2_d{dims[1]}", f"bwd_conv1_d{dims[0]}"]
    algo = [bytes_forward(n, e, dims[0]), bytes_forward(n, e, dims[1]),
            bytes_backward(n, dims[1], hp.path[1], src_rows[1]), bytes_backward(n, dims[0], hp.path[0], src_rows[0])]

    def step():
        hp.forward(ins[0], outs[0]); hp.forward(ins[1], outs[1])
        hp.backward(1, ins[2], outs[2]); hp.backward(0, ins[3], outs[3])

    stream = torch.cuda.current_stream()
    # -- whole-step timing (the clock sampler runs from the warm-up to the last per-kernel launch) ----
    with ClockSampler(local) as clocks:
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        torch.cuda.synchronize()
        ms_step = ev0.elapsed_time(ev1) / args.steps
        # -- per-kernel timing (same launches, one event pair each) ----------
        per = [[] for _ in range(4)]
        fns = [lambda: hp.forward(ins[0], outs[0]), lambda: hp.forward(ins[1], outs[1]),
               lambda: hp.backward(1, ins[2], outs[2]), lambda: hp.backward(0, ins[3], outs[3])]
        for _ in range(args.steps):
            for k, fn in enumerate(fns):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream); fn(); b.record(stream)
                per[k].append((a, b))
        torch.cuda.synchronize()
        # -- the bare gather of the two forward aggregations: the floor on this GPU -------
        floor = []
        sink = torch.zeros(1, device=dev)
        for k in range(2):
            evs = []
            for _ in range(max(5, args.steps // 2)):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream); probe_gather(hp.col, ins[k], sink); b.record(stream)
                evs.append((a, b))
            torch.cuda.synchronize()
            floor.append(statistics.mean(a.elapsed_time(b) for a, b in evs[2:]))
    kern_ms = [statistics.mean(a.elapsed_time(b) for a, b in p) for p in per]
    # the update step that produces the forward inputs (not part of the aggregation metric)
    x_in = torch.randn(n, spec["dim"], device=dev, generator=gen)
    w1 = torch.randn(spec["dim"], dims[0], device=dev, generator=gen)
    upd = []
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream); hp.capi.update_scaled(x_in, w1, hp.deg); b.record(stream)
        upd.append((a, b))
    torch.cuda.synchronize()
    update_ms = statistics.mean(a.elapsed_time(b) for a, b in upd[2:])
    del x_in
    peak, peak_src = measured_peak_gbs()
    kernels = {nm: {"ms": round(ms, 4), "algorithmic_mb": round(by / 1e6, 1), "gbs": round(by / ms / 1e6, 1),
                    "frac": round(by / ms / 1e6 / peak, 4)} for nm, ms, by in zip(names, kern_ms, algo)}
    kernels[f"update_k{spec['dim']}_d{dims[0]}"] = {
        "ms": round(update_ms, 4), "algorithmic_mb": round(4 * n * (spec["dim"] + dims[0]) / 1e6, 1),
        "gbs": round(4 * n * (spec["dim"] + dims[0]) / update_ms / 1e6, 1),
        "frac": round(4 * n * (spec["dim"] + dims[0]) / update_ms / 1e6 / peak, 4),
        "note": "diag(deg) (X W) with FP32 FMA; feeds the forward aggregation, outside the metric"}
    for k in range(2):
        row_bytes = ins[k].stride(0) * 4
        kernels[names[k]]["gather_floor_ms"] = round(floor[k], 4)
        kernels[names[k]]["gather_floor_tbs"] = round(e * row_bytes / floor[k] / 1e9, 2)
        kernels[names[k]]["of_gather_floor"] = round(floor[k] / kern_ms[k], 3)
    top = max(range(4), key=lambda k: kern_ms[k])
    roofline = {"bound": "hbm", "kernel": names[top], "achieved": round(algo[top] / kern_ms[top] / 1e6, 1),
                "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                "frac": round(algo[top] / kern_ms[top] / 1e6 / peak, 4), "traffic": None,
                "algorithmic_bytes": algo[top], "ms": round(kern_ms[top], 4)}
    if args.workload == "rmat21" and args.seed == 0:
        roofline["traffic"] = NCU_DRAM_TRAFFIC.get(names[top])
        roofline["traffic_note"] = "dram__bytes_read+write of one launch, ncu capture summarised under profiles/"

    # -- e2e: host buffers through the C-ABI ------------------------------------
    if args.kernels_only:
        print(json.dumps({"value": round(ms_step, 4), "kernels": kernels, "roofline": roofline}), flush=True)
        return
    host_in = [torch.empty(x.shape, pin_memory=True).copy_(x) for x in ins]
    host_out = [torch.empty(o.shape, pin_memory=True) for o in outs]
    stage = [padded(n, dims[0], dev, gen), padded(n, dims[1], dev, gen),
             torch.empty(n, dims[1], device=dev), torch.empty(n, dims[0], device=dev)]

    # Copies in, kernels and copies out run on three streams so that PCIe is busy in both directions
    # while the kernels run; events carry the dependencies, including the reuse of the staging buffers.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    staged_ev = [torch.cuda.Event() for _ in range(4)]      # H2D of input k finished
    done_ev = [torch.cuda.Event() for _ in range(4)]        # kernel k finished (input k reusable, output k ready)
    out_ev = [torch.cuda.Event() for _ in range(4)]         # D2H of output k finished (output k reusable)

    def e2e_step():
        for k in range(4):
            with torch.cuda.stream(s_in):
                s_in.wait_event(done_ev[k])
                stage[k].copy_(host_in[k], non_blocking=True)
                staged_ev[k].record(s_in)
            stream.wait_event(staged_ev[k])
            stream.wait_event(out_ev[k])
            (hp.forward(stage[k], outs[k]) if k < 2 else hp.backward(1 if k == 2 else 0, stage[k], outs[k]))
            done_ev[k].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done_ev[k])
                host_out[k].copy_(outs[k], non_blocking=True)
                out_ev[k].record(s_out)

    def e2e_join():
        stream.wait_stream(s_in)
        stream.wait_stream(s_out)

    for _ in range(2):
        e2e_step()
    e2e_join()
    torch.cuda.synchronize()
    e2e_steps = max(3, min(args.steps, 10))
    ev0.record(stream)
    s_in.wait_event(ev0)
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()
    ev1.record(stream)
    torch.cuda.synchronize()
    e2e_ms = ev0.elapsed_time(ev1) / e2e_steps
    h2d = sum(x.numel() * 4 for x in ins)
    d2h = sum(o.numel() * 4 for o in outs)

    # -- full training epoch through the operator module (context) --------------
    epoch_full = None
    if not args.no_full_epoch:
        from eppgcn_b200.train import GCNTrainer
        ds2 = graphs.load_workload(args.workload, args.seed)
        tr = GCNTrainer(ds2, hidden=spec["hidden"], backsize_mode="constant", backsize=args.backsize)
        for _ in range(3):
            tr.train_epoch()
        torch.cuda.synchronize()
        ev0.record(stream)
        for _ in range(args.steps):
            tr.train_epoch()
        ev1.record(stream)
        torch.cuda.synchronize()
        epoch_full = {"ms": round(ev0.elapsed_time(ev1) / args.steps, 4),
                      "what": "forward + log_softmax/nll_loss + backward + Adam through GCNConv, X resident"}
        del tr, ds2

    # -- CPU baseline on this box's host cores -------------------------------------
    cpu = None
    if not args.no_cpu_baseline:
        ms, cores, epochs = run_cpu(graph, dims, 5, 1, budget_s=20.0)
        cpu = {"value": round(ms, 2), "unit": "ms/epoch", "cores": cores, "kind": "port",
               "sample": f"{epochs} epoch(s) of the full workload: 4 torch.sparse CSR SpMMs over the whole graph"}

    line = {
        "metric": "2-layer GCN ms/epoch (fwd+bwd aggregation)", "value": round(ms_step, 4), "unit": "ms/epoch",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4),
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: R-MAT a=.57 b=.19 c=.19, N={n}, E={e} directed incl. self loops, "
                               f"dims {dims[0]}/{dims[1]}, train_ratio {spec['train_ratio']}, "
                               f"group size {hp.part_size}, backward part size {args.backsize}",
                   "seed": args.seed, "l2": "inputs exceed L2: each step streams >1 GB of distinct data",
                   "parallelism": "single GPU"},
        "kernels": kernels, "roofline": roofline, "clocks": clocks.summary(),
        "e2e": {"value": round(e2e_ms, 4), "unit": "ms/epoch", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "what": "same four aggregations through the C-ABI, inputs from pinned host memory, results copied back"},
        "gpu_launches": 4 * args.steps,
        "prep": {"build_part_s": round(hp.build_part_s, 3), "mask_compact_split_s": round(hp.prep_s, 4),
                 "active_edges": [p["valid"] for p in hp.path], "parts": [p["parts"] for p in hp.path]},
        "epoch_full": epoch_full, "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)


def run_reference(args):
    """CPU GCN path on the host cores; under torchrun only rank 0 works."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    from eppgcn_b200 import graphs
    spec = graphs.WORKLOADS[args.workload]
    if spec.get("draw") == "device":
        print(json.dumps({"impl": "reference", "unavailable": f"{args.workload} is drawn on the GPU (its host "
                          "generation takes too long for a bench run); the CPU arm covers the host-drawn workloads"}),
              flush=True)
        return
    graph = graphs.make_graph(args.workload, args.seed)
    dims = [spec["hidden"], spec["classes"]]
    ms, cores, epochs = run_cpu(graph, dims, args.steps, args.warmup, budget_s=90.0)
    line = {
        "impl": "reference", "metric": "2-layer GCN ms/epoch (fwd+bwd aggregation)", "value": round(ms, 2),
        "unit": "ms/epoch", "n_gpus": args.gpus, "steps": epochs, "warmup": min(args.warmup, 2),
        "ms_per_step": round(ms, 2), "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: N={graph.num_nodes}, E={graph.num_edges}, dims {dims[0]}/{dims[1]}",
                   "seed": args.seed, "parallelism": f"{cores} host threads"},
        "cpu_baseline": {"value": round(ms, 2), "unit": "ms/epoch", "cores": cores, "kind": "port",
                         "sample": f"{epochs} epoch(s) of the full workload: 4 torch.sparse CSR SpMMs over the "
                                   f"whole graph (the reference has no CPU implementation of its CUDA operators)"},
        "e2e": {"value": round(ms, 2), "unit": "ms/epoch", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="rmat21")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--backsize", type=int, default=32)
    p.add_argument("--exchange", default="balanced_halo", choices=["balanced", "allgather", "halo", "balanced_halo"],
                   help="multi-GPU partition/exchange, see eppgcn_b200.dist.DistHotPath")
    p.add_argument("--chunks", type=int, default=0,
                   help="balanced_halo: column chunks per exchange, one compact source buffer each; 0 = two when "
                        "every layer is at least 32 columns wide (and splits into 16-byte pieces), else one")
    p.add_argument("--overlap", action="store_true",
                   help="balanced_halo with the push transport and >1 chunk: push chunk c+1 on a side stream while "
                        "chunk c is aggregated (not yet measured; off by default)")
    p.add_argument("--transport", default="push", choices=["push", "nccl"],
                   help="balanced_halo: peer stores by this library's kernel, or NCCL all-to-all")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-full-epoch", action="store_true")
    p.add_argument("--kernels-only", action="store_true",
                   help="device-resident timing only (no e2e, full-epoch or CPU legs); for profiler captures")
    args = p.parse_args()
    if args.kernels_only:
        args.no_cpu_baseline = args.no_full_epoch = True
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
