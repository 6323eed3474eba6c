#!/usr/bin/env python
"""Benchmark of the GCN aggregation hot path.

Metric: ms per epoch of the forward + backward neighbour aggregation of a
2-layer GCN (hidden 16, 22 classes) -- two forward aggregations over the whole
graph and two backward aggregations over the prepared execution path -- on a
seeded R-MAT scale-21 graph (2,097,152 vertices, 35,651,584 directed edges with
self loops) unless another workload is named.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                  [--workload NAME] [--train-ratio R] [--kernel tiles|groups]

* ``value``  device-resident: inputs already in HBM, K steps timed with CUDA
  events around the C-ABI launches the operator module makes per epoch (the
  planned tile kernel; for a backward layer also the packing of its source
  rows and the clearing of the result).
* ``e2e``    the same four aggregations through the C-ABI with HOST buffers:
  every step copies its four input matrices from pinned host memory and
  copies the four results back.
* ``roofline``  the dominant kernel's compulsory bytes / its CUDA-event time,
  against the measured HBM copy bandwidth.
* ``check``  outside the timed region: every aggregation's result on sampled
  rows (the highest-degree rows among them) against the float64 oracle.
* ``ref_cuda``  the reference's own CUDA operators (unmodified build under
  oracle/_ref, when present) on the same workload, run in a child process.
* ``cpu_baseline`` / ``--impl reference``  the CPU GCN path (torch.sparse CSR
  SpMM, fp32, all host cores) on the same graph: the same four aggregations,
  over the whole graph in both directions (the CPU path has no execution-path
  preparation, so its backward is the uncompacted one).
"""
from __future__ import annotations

import argparse
import hashlib
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

METRIC = "2-layer GCN ms/epoch (fwd+bwd aggregation)"


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def measured_peak_gbs():
    """(GB/s, source) of the HBM roofline denominator."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


L2_FLUSH_BYTES = 256 << 20       # twice the 126 MB L2


def l2_policy(n, e, dims):
    """The ``config.l2`` wording of a workload (the same in both arms) and whether its forward inputs fit
    the flush size, in which case the GPU arm times every step behind a flush."""
    fits = min(bytes_forward(n, e, d) for d in dims[:2]) < L2_FLUSH_BYTES
    return ("L2 flushed (256 MiB written) before every timed step" if fits else
            "inputs exceed L2: every aggregation reads more than the 126 MB cache holds"), fits


def recorded_traffic(kernel_source: str):
    """DRAM bytes per launch from the committed profiler record, valid only while the kernel source it
    was captured at is unchanged: the record, or {}."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_dram_traffic.json")) as f:
            rec = json.load(f)
        with open(os.path.join(ROOT, "eppgcn_b200", "csrc", kernel_source), "rb") as f:
            digest = hashlib.sha1(f.read()).hexdigest()[:16]
        if rec.get("source") == kernel_source and rec.get("source_sha1_16") == digest:
            return rec
    except Exception:
        pass
    return {}


def workload_string(name, spec, n, e, dims, ratio, part_size, backsize):
    """One wording of the workload for both arms, so that their lines can be matched."""
    kind = "R-MAT a=.57 b=.19 c=.19" if spec["kind"] == "rmat" else f"Chung-Lu exponent {spec['exponent']}"
    return (f"{name}: {kind}, N={n}, E={e} directed incl. self loops, dims {'/'.join(str(d) for d in dims)}, "
            f"train_ratio {ratio}, group size {part_size}, backward part size {backsize}")


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
    one, spent = 1.0, 0.0
    for _ in range(max(1, warmup)):
        t0 = time.perf_counter()
        cpu_gcn.aggregation_epoch(a, mats)
        one = time.perf_counter() - t0
        spent += one
        if spent > budget_s / 3:             # a slow host: the warm-up is cut short
            break
    epochs = max(1, min(steps, int(budget_s / max(one, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(epochs):
        cpu_gcn.aggregation_epoch(a, mats)
    ms = (time.perf_counter() - t0) * 1e3 / epochs
    return ms, cores, epochs


def run_cpu_training(ds, spec, epochs):
    """Whole training epochs of the dense-update / sparse-aggregate GCN on the CPU (forward, loss on
    the train rows, backward, Adam), for the CPU-only configuration: ms/epoch."""
    from oracle import cpu_gcn
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    a = cpu_gcn.normalised_csr(ds.graph)
    g = torch.Generator().manual_seed(1)
    dims = [spec["dim"], spec["hidden"], spec["classes"]]
    weights = [torch.nn.Parameter((torch.rand(dims[i], dims[i + 1], generator=g) * 2 - 1) / dims[i + 1] ** 0.5)
               for i in range(2)]
    opt = torch.optim.Adam(weights, lr=0.01)
    x, y, mask = ds.x.cpu(), ds.y.cpu(), ds.train_mask.cpu()
    for _ in range(3):
        cpu_gcn.gcn_epoch(a, x, weights, y, mask, opt)
    t0 = time.perf_counter()
    for _ in range(epochs):
        cpu_gcn.gcn_epoch(a, x, weights, y, mask, opt)
    return (time.perf_counter() - t0) * 1e3 / epochs


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class HotPath:
    """Device-resident state of one GPU: CSR, groups, prepared path, aggregation plans."""

    def __init__(self, ds, dev, back_size=32, kernel="tiles"):
        import eppgcn_b200
        from eppgcn_b200 import capi
        self.capi, self.dev, self.kernel = capi, dev, kernel
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
        # plans of the tiled kernel, one per edge list (what the operator module builds at first use)
        self.plan_s = None
        if kernel == "tiles":
            t0 = time.perf_counter()
            self.fwd_plan = capi.TilePlan.from_csr(self.row, self.col)
            for p in self.path:
                p["plan"] = capi.TilePlan.from_ids(p["id"], p["edges"], p["valid"], n)
                p["src"] = {}
            torch.cuda.synchronize(dev)
            self.plan_s = time.perf_counter() - t0

    def forward(self, feat, out):
        """Forward aggregation as the operator module runs it: the update step has already folded
        deg[col] into the rows of `feat`."""
        if self.kernel == "tiles":
            return self.capi.spmm_tiles(feat, self.fwd_plan, self.deg, out=out)
        return self.capi.spmm_forward(feat, self.row, self.col, self.deg, self.pp, self.p2n, self.part_size, out=out,
                                      prescaled=True)

    def backward(self, i, d_out, out):
        """Backward aggregation of convolution i+1 as the operator module runs it: with the plan, the
        source rows are packed (scaled by deg, padded rows) and aggregated; else the group kernel."""
        p = self.path[i]
        if self.kernel == "tiles":
            d = d_out.size(1)
            if d not in p["src"]:
                p["src"][d] = torch.empty(self.n, (d + 7) // 8 * 8, device=self.dev)[:, :d]
            src = self.capi.pack_scaled_rows(d_out, self.deg, p["plan"], out=p["src"][d])
            return self.capi.spmm_tiles(src, p["plan"], self.deg, out=out)
        return self.capi.spmm_backward_compacted(d_out, p["id"], p["pp"], p["edges"], self.deg, p["parts"],
                                                 self.back_size, out=out)

    def launches_per_step(self):
        """This library's kernels in one epoch of four aggregations."""
        if self.kernel != "tiles":
            return 4
        k = 0
        for plan in (self.fwd_plan, self.fwd_plan):
            k += 1 + (1 if plan.info["cleared_rows"] and not plan.info["clears_whole_result"] else 0)
        for p in self.path:
            k += 2 + (1 if p["plan"].info["cleared_rows"] and not p["plan"].info["clears_whole_result"] else 0)
        return k


def padded(n, d, dev, gen):
    """[n, d] view with a row stride that is a multiple of 8 floats, as the forward operator lays out X @ W."""
    ld = (d + 7) // 8 * 8
    full = torch.randn(n, ld, device=dev, generator=gen)
    return full[:, :d]


def bytes_forward(n, e, d):
    return 4 * e + 4 * (n + 1) + 4 * n + 4 * d * n + 4 * d * n


def bytes_backward(n, d, p, src_rows):
    return 4 * p["valid"] + 4 * (p["parts"] + 1) + 4 * p["parts"] + 4 * d * src_rows + 4 * (p["rows"] + src_rows) + 4 * d * n


def sample_rows(indptr, count, seed):
    """Rows to check: the 1,000 rows with the most edges, then a seeded uniform sample."""
    n = len(indptr) - 1
    deg = np.diff(indptr)
    top = np.argsort(-deg, kind="stable")[:min(1000, n)]
    rng = np.random.Generator(np.random.PCG64(seed))
    rest = rng.choice(n, size=min(count, n), replace=False)
    return np.unique(np.concatenate([top, rest]))


def check_against_oracle(ds, hp, ins, outs, dims, rows_wanted=200_000):
    """Each of the four results on sampled rows against the float64 oracle.  The forward inputs are
    pre-scaled rows, so the oracle gets rows divided back by deg in float64; tolerance
    |got - want| <= 2e-6 + 2e-5 |want|.  Returns the `check` object of the bench line."""
    from oracle import epp_oracle as O
    ip, ix = ds.graph.indptr, ds.graph.indices
    deg = hp.deg.cpu().numpy().astype(np.float64)
    rows = sample_rows(ip, rows_wanted, 7)
    worst, detail = -np.inf, {}
    for k in range(4):
        x = ins[k].cpu().numpy().astype(np.float64)
        got = outs[k].cpu().numpy()[rows]
        if k < 2:
            want = O.spmm_rows(ip, ix, rows, x, row_scale=deg)                 # rows already carry deg[col]
        else:
            p = hp.path[1 if k == 2 else 0]
            v = p["valid"]
            want = O.spmm_rows_from_pairs(p["id"][:v].cpu().numpy(), p["edges"][:v].cpu().numpy(), hp.n, rows,
                                          x * deg[:, None], row_scale=deg)
        excess = float((np.abs(got - want) - (2e-6 + 2e-5 * np.abs(want))).max())
        worst = max(worst, excess)
        detail[("fwd_l1", "fwd_l2", "bwd_conv2", "bwd_conv1")[k]] = excess
    return {"rows": int(rows.size), "max_excess": worst, "ok": bool(worst <= 0),
            "tolerance": "|got-want| <= 2e-6 + 2e-5|want| against float64, sampled rows incl. the 1000 of highest degree",
            "per_aggregation": detail}


def ref_cuda_child(args):
    """Child process: the reference's own CUDA operators on the workload, timed by the reference's own
    event timers (for_agg_time / back_agg_time, EPPGCN_kernel.cu:96-116); prints one JSON object."""
    from eppgcn_b200 import graphs
    from oracle.ref_loader import load_reference
    ref = load_reference()
    if ref is None:
        print(json.dumps({"unavailable": "oracle/_ref holds no build of the reference's extension"}), flush=True)
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    spec = graphs.WORKLOADS[args.workload]
    ds = graphs.load_workload(args.workload, args.seed, train_ratio=args.train_ratio)
    hp = HotPath(ds, dev, args.backsize, kernel="groups")          # int32 metadata from this library's preparation
    n = hp.n
    dims = [spec["dim"], spec["hidden"], spec["classes"]]
    gen = torch.Generator(device=dev).manual_seed(args.seed)
    xs = [torch.randn(n, dims[i], device=dev, generator=gen) for i in range(2)]
    ws = [(torch.rand(dims[i], dims[i + 1], device=dev, generator=gen) - 0.5) / 2 for i in range(2)]
    douts = [torch.randn(n, dims[i + 1], device=dev, generator=gen) for i in range(2)]
    dim_worker = [min(dims[0], 32), min(dims[1], 32)]

    def epoch():
        for i in range(2):
            ref.forward(xs[i], ws[i], hp.row, hp.col, hp.deg, hp.pp, hp.p2n, hp.part_size, dim_worker[i], 8)
        for i in (1, 0):
            p = hp.path[i]
            ref.ours_backward(douts[i], xs[i], ws[i], p["id"], p["pp"], p["edges"], hp.deg, hp.back_size, p["parts"],
                              i + 1, 4, 16)

    for _ in range(2):
        epoch()
    torch.cuda.synchronize()
    ref.clear_time()
    epochs = max(3, min(args.steps, 10))
    for _ in range(epochs):
        epoch()
    torch.cuda.synchronize()
    # the reference prints its timers with printf: catch file descriptor 1
    sys.stdout.flush()
    r, w = os.pipe()
    saved = os.dup(1)
    os.dup2(w, 1)
    try:
        ref.print_time()
        import ctypes
        ctypes.CDLL(None).fflush(None)
    finally:
        os.dup2(saved, 1)
        os.close(w)
    text = os.read(r, 1 << 16).decode()
    os.close(r)
    vals = {}
    for line in text.splitlines():
        if ":" in line:
            key, _, v = line.partition(":")
            try:
                vals[key.strip()] = float(v)
            except ValueError:
                pass
    fwd, bwd = vals.get("for_agg_time"), vals.get("back_agg_time")
    if fwd is None or bwd is None:
        print(json.dumps({"unavailable": f"could not read the reference's timers: {text!r}"}), flush=True)
        return
    print(json.dumps({"ms_per_epoch": round((fwd + bwd) * 1e3 / epochs, 4),
                      "forward_ms": round(fwd * 1e3 / epochs, 4), "backward_ms": round(bwd * 1e3 / epochs, 4),
                      "per_layer_backward_ms": {k: round(v * 1e3 / epochs, 4) for k, v in vals.items()
                                                if k.startswith("l") and k.endswith("_back_agg_time")},
                      "epochs": epochs, "workload": args.workload,
                      "what": "the reference's spmm_forward_cuda_kernel and ours_backward_cuda_kernel (unmodified "
                              "sources compiled for sm_100), its own event timers, same graph, seed, masks and "
                              "int32 partition metadata"}), flush=True)


def run_ref_cuda(args, timeout_s=240):
    """Runs the reference-kernel leg in a child process, so that nothing it does can take the bench down."""
    if not os.path.isdir(os.path.join(ROOT, "oracle", "_ref")):
        return {"unavailable": "oracle/_ref holds no build of the reference's extension"}
    cmd = [sys.executable, os.path.abspath(__file__), "--ref-cuda-child", "--workload", args.workload, "--seed",
           str(args.seed), "--backsize", str(args.backsize), "--steps", str(args.steps)]
    if args.train_ratio is not None:
        cmd += ["--train-ratio", str(args.train_ratio)]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference-kernel leg did not finish within {timeout_s} s"}
    for line in reversed(r.stdout.splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                break
    return {"unavailable": f"the reference-kernel leg exited with code {r.returncode}: {r.stderr[-300:]!r}"}


def run_gpu(args):
    from eppgcn_b200 import graphs
    rank = int(os.environ.get("RANK", 0)); world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    spec = graphs.WORKLOADS[args.workload]
    if world > 1 or spec.get("draw") == "device":
        # several ranks, or a workload that is drawn on the GPU: the row-partitioned driver (also at one rank)
        import bench_multi
        return bench_multi.run_bench(args, rank, world, dev)

    ratio = spec["train_ratio"] if args.train_ratio is None else args.train_ratio
    t0 = time.perf_counter()
    ds = graphs.load_workload(args.workload, args.seed, train_ratio=args.train_ratio)
    log(f"[bench] workload {args.workload}: N={ds.num_nodes} E={ds.num_edges} ({time.perf_counter() - t0:.1f}s)")
    graph = ds.graph
    n, e = ds.num_nodes, ds.num_edges
    dims = [spec["hidden"], spec["classes"]]
    hp = HotPath(ds, dev, args.backsize, args.kernel)
    src_rows = [int(ds.ngh_masks[0].sum().item()), int(ds.train_mask.sum().item())]   # conv1, conv2
    gen = torch.Generator(device=dev).manual_seed(args.seed)
    ins = [padded(n, dims[0], dev, gen), padded(n, dims[1], dev, gen),
           torch.randn(n, dims[1], device=dev, generator=gen), torch.randn(n, dims[0], device=dev, generator=gen)]
    outs = [torch.empty(n, d, device=dev) for d in (dims[0], dims[1], dims[1], dims[0])]
    names = [f"fwd_d{dims[0]}", f"fwd_d{dims[1]}", f"bwd_conv2_d{dims[1]}", f"bwd_conv1_d{dims[0]}"]
    algo = [bytes_forward(n, e, dims[0]), bytes_forward(n, e, dims[1]),
            bytes_backward(n, dims[1], hp.path[1], src_rows[1]), bytes_backward(n, dims[0], hp.path[0], src_rows[0])]
    fns = [lambda: hp.forward(ins[0], outs[0]), lambda: hp.forward(ins[1], outs[1]),
           lambda: hp.backward(1, ins[2], outs[2]), lambda: hp.backward(0, ins[3], outs[3])]

    def step():
        for fn in fns:
            fn()

    stream = torch.cuda.current_stream()
    # Every aggregation of the large workloads reads more than the L2 holds; a small graph would stay
    # cached from one step to the next, so its steps are timed one by one behind a 256 MiB write.
    l2_note, fits = l2_policy(n, e, dims)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev) if fits else None
    # -- whole-step timing (the clock sampler runs from the warm-up to the last per-kernel launch) ----
    with ClockSampler(local) as clocks:
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if flush is None:
            torch.cuda.synchronize()
            ev0.record(stream)
            for _ in range(args.steps):
                step()
            ev1.record(stream)
            torch.cuda.synchronize()
            ms_step = ev0.elapsed_time(ev1) / args.steps
        else:                       # a workload that fits L2: every step starts from a flushed cache
            pairs = []
            for _ in range(args.steps):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream); step(); b.record(stream)
                pairs.append((a, b))
            torch.cuda.synchronize()
            ms_step = statistics.mean(a.elapsed_time(b) for a, b in pairs)
        # -- per-aggregation timing (same launches, one event pair each) ----------
        per = [[] for _ in range(4)]
        for _ in range(args.steps):
            for k, fn in enumerate(fns):
                if flush is not None:
                    flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream); fn(); b.record(stream)
                per[k].append((a, b))
        torch.cuda.synchronize()
        # -- the bare gather of the two forward aggregations, in CSR order --------
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
    upd_bytes = 4 * n * (spec["dim"] + dims[0])
    kernels[f"update_k{spec['dim']}_d{dims[0]}"] = {
        "ms": round(update_ms, 4), "algorithmic_mb": round(upd_bytes / 1e6, 1),
        "gbs": round(upd_bytes / update_ms / 1e6, 1), "frac": round(upd_bytes / update_ms / 1e6 / peak, 4),
        "note": "diag(deg) (X W) with FP32 FMA; feeds the forward aggregation, outside the metric"}
    for k in range(2):
        row_bytes = ins[k].stride(0) * 4
        kernels[names[k]]["csr_order_gather_ms"] = round(floor[k], 4)
        kernels[names[k]]["csr_order_gather_tbs"] = round(e * row_bytes / floor[k] / 1e9, 2)
    top = max(range(4), key=lambda k: kern_ms[k])
    traffic = recorded_traffic("tiled_spmm.cu") if args.kernel == "tiles" else {}
    roofline = {"bound": "hbm", "kernel": names[top], "achieved": round(algo[top] / kern_ms[top] / 1e6, 1),
                "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                "frac": round(algo[top] / kern_ms[top] / 1e6 / peak, 4), "traffic": None,
                "algorithmic_bytes": algo[top], "ms": round(kern_ms[top], 4)}
    if traffic.get("workload") == args.workload and traffic.get("seed") == args.seed and ratio == spec["train_ratio"]:
        roofline["traffic"] = traffic.get("dram_bytes_per_launch", {}).get(names[top])
        roofline["traffic_note"] = "dram__bytes_read+write of one aggregation from the recorded ncu capture of this source"

    if args.kernels_only:
        print(json.dumps({"value": round(ms_step, 4), "kernels": kernels, "roofline": roofline}), flush=True)
        return
    # -- parity at the size that was timed (outside the timed region) -----------------
    check = None
    if not args.no_check:
        step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        check = check_against_oracle(ds, hp, ins, outs, dims)
        check["seconds"] = round(time.perf_counter() - t0, 1)
        log(f"[bench] check: {check}")

    # -- e2e: host buffers through the C-ABI ------------------------------------
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
    del host_in, host_out, stage

    # -- full training epoch through the operator module (context) --------------
    epoch_full = None
    if not args.no_full_epoch:
        from eppgcn_b200.train import GCNTrainer
        ds2 = graphs.load_workload(args.workload, args.seed, train_ratio=args.train_ratio)
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

    # -- the reference's own kernels on this GPU, in a child process -----------------
    ref_cuda = None
    if not args.no_ref_cuda:
        torch.cuda.empty_cache()
        ref_cuda = run_ref_cuda(args)
        log(f"[bench] ref_cuda: {ref_cuda}")

    # -- CPU baseline on this box's host cores -------------------------------------
    cpu = None
    if not args.no_cpu_baseline:
        ms, cores, epochs = run_cpu(graph, dims, 5, 1, budget_s=20.0)
        cpu = {"value": round(ms, 2), "unit": "ms/epoch", "cores": cores, "kind": "port",
               "sample": f"{epochs} epoch(s) of the full workload: 4 torch.sparse CSR SpMMs over the whole graph "
                         f"(the CPU path has no execution-path preparation: its backward is the uncompacted one)"}

    active = [p["valid"] for p in hp.path]
    line = {
        "metric": METRIC, "value": round(ms_step, 4), "unit": "ms/epoch",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4),
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_string(args.workload, spec, n, e, dims, ratio, hp.part_size, args.backsize),
                   "seed": args.seed, "l2": l2_note,
                   "parallelism": "single GPU",
                   "kernel": "tiled plan (rows in width classes, padded edge copy)" if args.kernel == "tiles"
                             else "neighbour-group kernel"},
        "kernels": kernels, "roofline": roofline, "clocks": clocks.summary(), "check": check,
        "e2e": {"value": round(e2e_ms, 4), "unit": "ms/epoch", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "what": "same four aggregations through the C-ABI, inputs from pinned host memory, results copied back"},
        "gpu_launches": hp.launches_per_step() * args.steps,
        "prep": {"build_part_s": round(hp.build_part_s, 3), "mask_compact_split_s": round(hp.prep_s, 4),
                 "aggregation_plans_s": None if hp.plan_s is None else round(hp.plan_s, 3),
                 "active_edges": active, "active_edge_share": [round(v / e, 4) for v in active],
                 "parts": [p["parts"] for p in hp.path]},
        "epoch_full": epoch_full, "ref_cuda": ref_cuda, "cpu_baseline": cpu,
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
    ds = graphs.load_workload(args.workload, args.seed, train_ratio=args.train_ratio)
    graph = ds.graph
    ratio = spec["train_ratio"] if args.train_ratio is None else args.train_ratio
    dims = [spec["hidden"], spec["classes"]]
    warm = max(args.warmup, 3)
    ms, cores, epochs = run_cpu(graph, dims, args.steps, warm, budget_s=90.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(ms, 2),
        "unit": "ms/epoch", "n_gpus": args.gpus, "steps": args.steps, "warmup": warm,
        "ms_per_step": round(ms, 2), "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_string(args.workload, spec, graph.num_nodes, graph.num_edges, dims, ratio,
                                               max(int(ds.avg_degree), 1), args.backsize),
                   "seed": args.seed, "l2": l2_policy(graph.num_nodes, graph.num_edges, dims)[0],
                   "parallelism": "single GPU",
                   "kernel": "tiled plan (rows in width classes, padded edge copy)" if args.kernel == "tiles"
                             else "neighbour-group kernel"},
        "arm": {"host_threads": cores, "epochs_timed": epochs,
                "what": "fp32 torch.sparse CSR SpMM on the host cores; four whole-graph aggregations per epoch: "
                        "the CPU path has no execution-path preparation, so its backward is the uncompacted one "
                        "(the GPU arm's backward runs over the compacted path)"},
        "cpu_baseline": {"value": round(ms, 2), "unit": "ms/epoch", "cores": cores, "kind": "port",
                         "sample": f"{epochs} epoch(s) of the full workload: 4 torch.sparse CSR SpMMs over the "
                                   f"whole graph (the reference has no CPU implementation of its CUDA operators)"},
        "e2e": {"value": round(ms, 2), "unit": "ms/epoch", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if args.cpu_training_epochs > 0:
        line["cpu_training"] = {"ms_per_epoch": round(run_cpu_training(ds, spec, args.cpu_training_epochs), 3),
                                "epochs": args.cpu_training_epochs, "cores": cores,
                                "what": "whole training epochs on the CPU: forward, loss on the train rows, "
                                        "backward, Adam (the CPU-only configuration)"}
    print(json.dumps(line), flush=True)


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="rmat21")
    p.add_argument("--train-ratio", type=float, default=None, help="train mask ratio (default: the workload's own)")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--backsize", type=int, default=32)
    p.add_argument("--kernel", default="tiles", choices=["tiles", "groups"],
                   help="single GPU: the planned tile kernel the operator module uses, or the stateless group kernel")
    p.add_argument("--exchange", default="balanced_halo", choices=["balanced", "allgather", "halo", "balanced_halo"],
                   help="multi-GPU partition/exchange, see eppgcn_b200.dist.DistHotPath")
    p.add_argument("--chunks", type=int, default=0,
                   help="balanced_halo: column chunks per exchange, one compact source buffer each; 0 = two when "
                        "every layer is at least 32 columns wide (and splits into 16-byte pieces), else one")
    p.add_argument("--overlap", action="store_true",
                   help="balanced_halo with the push transport and >1 chunk: push chunk c+1 on a side stream while "
                        "chunk c is aggregated")
    p.add_argument("--transport", default="push", choices=["push", "nccl"],
                   help="balanced_halo: peer stores by this library's kernel, or NCCL all-to-all")
    p.add_argument("--lead-barrier", action="store_true",
                   help="balanced_halo, push transport: always wait for the readers of a buffer before pushing into "
                        "it (default: only when no other barrier has passed since it was read)")
    p.add_argument("--stream", action="store_true",
                   help="multi-GPU, push transport: push the rows peer by peer on a side stream while the edges of the "
                        "owners that have landed are aggregated (default: push everything, one barrier, then aggregate)")
    p.add_argument("--owner-groups", type=int, default=0,
                   help="multi-GPU streamed exchange: bundle the other ranks' rows into this many groups (0: one per rank)")
    p.add_argument("--no-graph", action="store_true",
                   help="multi-GPU: submit every launch of the timed epoch by itself instead of replaying one CUDA graph")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-full-epoch", action="store_true")
    p.add_argument("--no-check", action="store_true")
    p.add_argument("--no-ref-cuda", action="store_true")
    p.add_argument("--cpu-training-epochs", type=int, default=0,
                   help="--impl reference: also time this many whole training epochs on the CPU")
    p.add_argument("--kernels-only", action="store_true",
                   help="device-resident timing only (no check, e2e, full-epoch, reference-kernel or CPU legs); "
                        "for profiler captures")
    p.add_argument("--ref-cuda-child", action="store_true", help=argparse.SUPPRESS)
    args = p.parse_args()
    if args.kernels_only:
        args.no_cpu_baseline = args.no_full_epoch = args.no_check = args.no_ref_cuda = True
    if args.ref_cuda_child:
        ref_cuda_child(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
