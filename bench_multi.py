"""Multi-GPU arm of bench.py (also used at one rank for workloads that are drawn on the GPU).

One process per GPU; the row-partitioned hot path itself lives in
``eppgcn_b200.dist``, this file only drives and times it and prints the
benchmark's JSON line on rank 0.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist

import bench as B
from eppgcn_b200 import graphs
from eppgcn_b200.dist import DistHotPath, DealtHalo  # noqa: F401  (DealtHalo: plan type of the default mode)


def count_launches(hp, step):
    """Runs one step with the C-ABI wrappers of ``hp.capi`` counting the kernels they enqueue: one per
    call, plus the row-clearing kernel of a tiled aggregation whose plan lists rows to clear (a plan
    that clears the whole result uses a memset, which is not a kernel), plus the clearing kernel of a
    group-kernel call that writes a column block."""
    capi = hp.capi
    names = ["push_rows", "peer_barrier", "peer_barrier_counted", "push_rows_signal", "bump_counter", "wait_landed",
             "spmm_tiles", "spmm_tiles_add", "pack_scaled_rows", "spmm_forward", "spmm_backward_compacted"]
    saved = {n: getattr(capi, n) for n in names}
    count = [0]

    def wrap(name, fn):
        def counted(*a, **k):
            count[0] += 1
            if name == "spmm_tiles":
                info = a[1].info
                count[0] += 1 if info["cleared_rows"] and not info["clears_whole_result"] else 0
            elif name in ("spmm_forward", "spmm_backward_compacted"):
                out = k.get("out")
                count[0] += 1 if out is not None and out.dim() == 2 and out.stride(0) != out.size(1) else 0
            return fn(*a, **k)
        return counted

    for n in names:
        setattr(capi, n, wrap(n, saved[n]))
    try:
        step()
        torch.cuda.synchronize()
    finally:
        for n in names:
            setattr(capi, n, saved[n])
    return count[0]


def check_shard(hp, ops, staged, local_in, outs, one, dev, rank, world, rows_wanted=50_000):
    """Runs every aggregation of the epoch once more and compares this rank's result rows (a sample
    that includes its 500 rows of highest degree) with the float64 oracle over the rank's shard of
    the relabelled graph and the inputs of all ranks.  Forward inputs are pre-scaled rows
    (out = deg[r] * sum x[c]); backward inputs are raw (out = deg[r] * sum deg[c] * x[c]).
    Tolerance |got - want| <= 2e-6 + 2e-5 |want|.  Returns the `check` object (the worst rank's)."""
    from oracle import epp_oracle as O
    sh = hp.shard
    ip = np.asarray(sh.indptr, dtype=np.int64)
    ix = np.asarray(sh.indices)
    deg = hp.deg.cpu().numpy().astype(np.float64)
    deg_row = deg[sh.v0:sh.v1]
    n_loc = hp.n_loc
    lens = np.diff(ip)
    top = np.argsort(-lens, kind="stable")[:min(500, n_loc)]
    rng = np.random.Generator(np.random.PCG64(11 + rank))
    rows = np.unique(np.concatenate([top, rng.choice(n_loc, size=min(rows_wanted, n_loc), replace=False)]))
    worst, detail = -np.inf, {}
    for k, (kind, i, d) in enumerate(ops):
        mine = torch.cat([v for v in staged[k]], dim=1).contiguous() if local_in[k] is None else local_in[k].contiguous()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        x = torch.cat(parts, dim=0).cpu().numpy().astype(np.float64)           # rows in the partition's numbering
        one(k)
        torch.cuda.synchronize()
        got = outs[k].cpu().numpy()[rows]
        if kind == "fwd":
            want = O.spmm_rows(ip, ix, rows, x, row_scale=deg_row)
        else:
            p = hp.path[i]
            v = p["valid"]
            want = O.spmm_rows_from_pairs(p["id"][:v].cpu().numpy(), p["edges"][:v].cpu().numpy(), n_loc, rows,
                                          x * deg[:x.shape[0], None], row_scale=deg_row)
        excess = float((np.abs(got - want) - (2e-6 + 2e-5 * np.abs(want))).max())
        detail[f"{kind}_l{i + 1}"] = excess
        worst = max(worst, excess)
    t = torch.tensor([worst], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if hp.fabric is not None:
        hp.fabric.check()
    return {"rows_per_rank": int(rows.size), "max_excess": float(t.item()), "ok": bool(t.item() <= 0),
            "tolerance": "|got-want| <= 2e-6 + 2e-5|want| against float64 on every rank's sampled rows",
            "rank0_per_aggregation": detail}


def check_shard_on_device(hp, ops, staged, local_in, outs, one, dev, rank, world):
    """The parity check of a workload that is drawn on the GPU and too large for the host oracle: every
    aggregation of the epoch is run once more and ALL of this rank's result rows are compared with a float64
    sparse product computed on the device by torch (cuSPARSE) from the rank's own CSR shard / compacted edge
    list and the input rows of all ranks -- an implementation that shares nothing with this library's
    kernels or exchange.  Tolerance |got - want| <= 2e-6 + 2e-5 |want|.  Returns the `check` object."""
    n_loc, n = hp.n_loc, hp.n
    deg = hp.deg.double()
    deg_row = hp.deg_row.double()
    worst, detail = -float("inf"), {}
    fwd = torch.sparse_csr_tensor(hp.row, hp.col, torch.ones(hp.col.numel(), dtype=torch.float64, device=dev),
                                  size=(n_loc, n))
    for k, (kind, i, d) in enumerate(ops):
        mine = torch.cat([v for v in staged[k]], dim=1).contiguous() if local_in[k] is None else local_in[k].contiguous()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        x = torch.cat(parts, dim=0).double()                       # rows in the partition's numbering
        del parts
        one(k)
        torch.cuda.synchronize()
        if kind == "fwd":
            want = torch.sparse.mm(fwd, x)
        else:
            p = hp.path[i]
            v = p["valid"]
            back = torch.sparse_coo_tensor(torch.stack([p["id"][:v].long(), p["edges"][:v].long()]),
                                           torch.ones(v, dtype=torch.float64, device=dev), size=(n_loc, n))
            want = torch.sparse.mm(back.coalesce(), x * deg[:x.size(0), None])
            del back
        want *= deg_row[:, None]
        excess = float(((outs[k].double() - want).abs() - (2e-6 + 2e-5 * want.abs())).max().item())
        del want, x
        detail[f"{kind}_l{i + 1}"] = excess
        worst = max(worst, excess)
    del fwd
    torch.cuda.empty_cache()
    t = torch.tensor([worst], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if hp.fabric is not None:
        hp.fabric.check()
    return {"rows_per_rank": int(n_loc), "max_excess": float(t.item()), "ok": bool(t.item() <= 0),
            "tolerance": "|got-want| <= 2e-6 + 2e-5|want| against a float64 cuSPARSE product on the device, every "
                         "row of every rank",
            "rank0_per_aggregation": detail}


def run_bench(args, rank: int, world: int, dev):
    """Multi-GPU arm of bench.py: the forward and backward aggregations of every
    layer, row-partitioned, each preceded by the exchange of its source rows.
    Strong scaling: the graph is fixed and split over the ranks.  Workloads whose
    ``WORKLOADS`` entry is too large for the host generator are drawn on the GPU
    (every rank draws the same graph from the same seed)."""
    if not dist.is_initialized():
        # NCCL announces its version on the process's standard output when the communicator is made; the only
        # line this program may print there is the result, so the descriptor points at standard error meanwhile
        import sys
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            if "MASTER_ADDR" in os.environ:
                dist.init_process_group("nccl", device_id=dev)
            else:       # plain `python bench.py` with a device-drawn workload: a group of one
                dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29533", rank=0, world_size=1,
                                        device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            os.dup2(saved, 1)
            os.close(saved)
    spec = graphs.WORKLOADS[args.workload]
    device_drawn = spec.get("draw") == "device"
    t0 = time.perf_counter()
    if device_drawn:
        ds = graphs.DeviceWorkload(args.workload, args.seed, dev)
    else:
        if rank == 0:
            ds = graphs.load_workload(args.workload, args.seed)      # generates and caches the graph once per box
        dist.barrier()
        if rank != 0:
            ds = graphs.load_workload(args.workload, args.seed)
    n, e, L = ds.num_nodes, ds.num_edges, ds.num_layers
    dims = [spec["hidden"]] * (L - 1) + [spec["classes"]]
    mode = getattr(args, "exchange", "balanced")
    if device_drawn and mode not in ("balanced", "balanced_halo"):
        mode = "balanced"
    halo = mode in ("halo", "balanced_halo")
    chunks = getattr(args, "chunks", 0)
    if chunks <= 0:           # measured on the 64/64/32-column workload: two 32-column buffers aggregate faster than one
        chunks = 2 if min(dims) >= 32 and all(d % 8 == 0 for d in dims) else 1
    hp = DistHotPath(ds, dev, rank, world, args.backsize, exchange=mode, chunks=chunks,
                     transport=getattr(args, "transport", "push"), overlap=getattr(args, "overlap", False),
                     streamed=getattr(args, "stream", False), owner_groups=getattr(args, "owner_groups", 0))
    dealt = mode == "balanced_halo"
    if dealt and getattr(args, "lead_barrier", False):
        for plan in [hp.fwd_plan] + [p["plan"] for p in hp.path]:
            plan.lead_barrier = True
    if device_drawn:
        ds.indptr = ds.indices = None           # the shard is all this rank needs from here on
        torch.cuda.empty_cache()
    setup_s = time.perf_counter() - t0
    n_loc = hp.n_loc
    gen = torch.Generator(device=dev).manual_seed(args.seed + rank)
    # operations of one epoch: forward of every layer, then backward from the last layer down
    ops = [("fwd", i, dims[i]) for i in range(L)] + [("bwd", i, dims[i]) for i in reversed(range(L))]
    # forward inputs as the update step leaves them (padded rows), backward inputs as autograd does (dense)
    if dealt:
        # forward: the producer (the update step) writes this rank's pre-scaled rows straight into the
        # exchange buffers; backward: the rows come from autograd, unscaled, in a matrix of their own, and
        # are multiplied by deg while they are copied into place
        local_in = [None if kind == "fwd" else torch.randn(n_loc, d, device=dev, generator=gen) for kind, _, d in ops]
        staged = [hp.halo_inputs(kind, i, d) if kind == "fwd" else [local_in[k]] for k, (kind, i, d) in enumerate(ops)]
        for views in staged:
            for v in views:
                v.normal_(generator=gen)
    else:
        local_in = [B.padded(n_loc, d, dev, gen) if kind == "fwd" else torch.randn(n_loc, d, device=dev, generator=gen)
                    for kind, _, d in ops]
        staged = [[x] for x in local_in]
    outs = [torch.empty(n_loc, d, device=dev) for _, _, d in ops]
    compact_bwd = "plan" in hp.path[0]
    full = [None] * len(ops)
    bufs = [None] * len(ops)
    for k, (kind, i, d) in enumerate(ops):
        if dealt:
            continue                                  # the plans keep their own per-aggregation buffers
        if halo:
            bufs[k] = (hp.fwd_plan if kind == "fwd" else hp.path[i]["plan"]).exchange(local_in[k])
        elif kind == "bwd" and compact_bwd:
            bufs[k] = hp.path[i]["plan"].exchange(local_in[k])
        else:
            full[k] = B.padded(hp.n, d, dev, gen) if kind == "fwd" else torch.empty(hp.n, d, device=dev)

    def one(k):
        kind, i, d = ops[k]
        if kind == "bwd" and (compact_bwd or halo):
            hp.backward_halo(i, local_in[k], outs[k])
        elif halo:
            hp.forward_halo(local_in[k], outs[k])
        else:
            hp.gather(full[k], local_in[k])
            (hp.forward(full[k], outs[k]) if kind == "fwd" else hp.backward(i, full[k], outs[k]))

    def local_only(k):
        kind, i, d = ops[k]
        if dealt:
            return hp.halo_local(kind, i, outs[k])
        if kind == "fwd":
            if not halo:
                return hp.forward(full[k], outs[k])
            return hp.capi.spmm_forward(bufs[k], hp.row, hp.col_c, hp.deg, hp.pp, hp.p2n, hp.part_size,
                                        out=outs[k], deg_row=hp.deg_row, prescaled=True)
        if not compact_bwd:
            return hp.backward(i, full[k], outs[k])
        p = hp.path[i]
        return hp.capi.spmm_backward_compacted(bufs[k], p["id"], p["pp"], p["edges_c"], p["deg_c"], p["parts"],
                                               hp.back_size, out=outs[k], deg_row=hp.deg_row, num_rows=n_loc)

    def step():
        for k in range(len(ops)):
            one(k)

    # this library's kernels per epoch, counted on one untimed step by wrapping the C-ABI calls
    launches_per_step = count_launches(hp, step)
    # The timed step is one CUDA graph of those launches (peer stores and flag barriers included) unless
    # --no-graph is given: a dozen small submissions per aggregation otherwise let the ranks drift apart on
    # the host, and every barrier then waits for the slowest submitter.
    graphed = dealt and not getattr(args, "no_graph", False) and (world == 1 or hp.fabric is not None)
    run = step
    if graphed:
        try:
            run = hp.graphed(step)
        except Exception as exc:              # noqa: BLE001 - any capture failure means "submit the launches one by one"
            B.log(f"[bench] rank {rank}: graph capture failed ({exc!r}); timing separate submissions")
            run = step
        # every rank replays the same thing: if the capture failed anywhere, nobody uses a graph
        agreed = torch.tensor([0 if run is step else 1], device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            run, graphed = step, False

    stream = torch.cuda.current_stream()
    with B.ClockSampler(dev.index) as clocks:
        for _ in range(max(args.warmup, 3)):
            run()
        torch.cuda.synchronize()
        if hp.fabric is not None:
            hp.fabric.check()
        dist.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        dist.barrier()
        ev0.record(stream)
        for _ in range(args.steps):
            run()
        ev1.record(stream)
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([ev0.elapsed_time(ev1) / args.steps], device=dev)
        # kernel-only share: the local SpMMs without the exchange
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(stream)
        for _ in range(args.steps):
            for k in range(len(ops)):
                local_only(k)
        k1.record(stream)
        torch.cuda.synchronize()
        kms = torch.tensor([k0.elapsed_time(k1) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    dist.all_reduce(kms, op=dist.ReduceOp.MAX)
    if hp.fabric is not None:
        hp.fabric.check()

    # parity of what was timed, outside the timed region: every aggregation's local result on sampled
    # rows against the float64 oracle of this rank's shard (host-drawn workloads), or on all rows against a
    # float64 sparse product on the device (the device-drawn graph is too large for a host oracle)
    check = None
    if mode in ("balanced", "balanced_halo") and not getattr(args, "no_check", False):
        check = (check_shard_on_device if device_drawn else check_shard)(hp, ops, staged, local_in, outs, one, dev,
                                                                         rank, world)

    # e2e: host buffers, every step stages this rank's rows in and its results out
    host_in = [[torch.empty(x.shape, pin_memory=True).copy_(x) for x in views] for views in staged]
    host_out = [torch.empty(o.shape, pin_memory=True) for o in outs]

    # Copies in, kernels and copies out run on three streams, so that PCIe is busy in both directions while
    # the exchange and the kernels run; events carry the dependencies, including the reuse of the staging
    # rows (an aggregation's input rows are overwritten only after the kernels that read them).
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    nops = len(ops)
    staged_ev = [torch.cuda.Event() for _ in range(nops)]
    done_ev = [torch.cuda.Event() for _ in range(nops)]
    out_ev = [torch.cuda.Event() for _ in range(nops)]

    def e2e_step():
        for k in range(nops):
            with torch.cuda.stream(s_in):
                s_in.wait_event(done_ev[k])
                for x, h in zip(staged[k], host_in[k]):
                    x.copy_(h, non_blocking=True)
                staged_ev[k].record(s_in)
            stream.wait_event(staged_ev[k])
            stream.wait_event(out_ev[k])
            one(k)
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
    dist.barrier()
    steps2 = max(3, min(args.steps, 10))
    ev0.record(stream)
    s_in.wait_event(ev0)
    for _ in range(steps2):
        e2e_step()
    e2e_join()
    ev1.record(stream)
    torch.cuda.synchronize()
    e2e = torch.tensor([ev0.elapsed_time(ev1) / steps2], device=dev)
    dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    byts = torch.tensor([sum(x.numel() * 4 for views in staged for x in views), sum(o.numel() * 4 for o in outs)],
                        device=dev, dtype=torch.int64)
    dist.all_reduce(byts)
    edges = torch.tensor([hp.shard.num_edges, n_loc], device=dev, dtype=torch.int64)
    gathered = [torch.zeros_like(edges) for _ in range(world)]
    dist.all_gather(gathered, edges)
    if rank == 0:
        peak, peak_src = B.measured_peak_gbs()
        exchanged = [(bufs[k].size(0) if bufs[k] is not None else hp.n) for k in range(len(ops))]
        if dealt:
            exchanged = [(hp.fwd_plan if kind == "fwd" else hp.path[i]["plan"]).num_remote for kind, i, _ in ops]
        # compulsory bytes of rank 0's local aggregations (each input byte once, each output byte once)
        e_loc = hp.shard.num_edges
        algo = 0
        for k, (kind, i, d) in enumerate(ops):
            if kind == "fwd":
                algo += 4 * e_loc + 4 * (n_loc + 1) + 4 * n_loc + 4 * d * min(exchanged[k] + n_loc, hp.n) + 4 * d * n_loc
            else:
                p = hp.path[i]
                src_rows = min(exchanged[k] + n_loc, hp.n)
                algo += (4 * p["valid"] + 4 * (p["parts"] + 1) + 4 * p["parts"] + 4 * d * src_rows
                         + 4 * (p["rows"] + src_rows) + 4 * d * n_loc)
        achieved = algo / (kms.item() * 1e-3) / 1e9
        launches = launches_per_step
        line = {
            "metric": f"{L}-layer GCN ms/epoch (fwd+bwd aggregation)", "value": round(ms.item(), 4),
            "unit": "ms/epoch", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms.item(), 4), "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: N={n}, E={e} directed incl. self loops, dims "
                                   f"{'/'.join(str(d) for d in dims)}, train_ratio {spec['train_ratio']}, "
                                   f"group size {hp.part_size}, backward part size {args.backsize}"
                                   + (", graph drawn on the GPU" if device_drawn else ""),
                       "seed": args.seed, "l2": "inputs exceed L2",
                       "parallelism": f"rows{world}: "
                                      + {"halo": "contiguous ranges, one NCCL all-to-all of the referenced source "
                                                 "rows per aggregation",
                                         "allgather": "contiguous ranges, one uneven NCCL row all-gather per aggregation",
                                         "balanced_halo": "degree-dealt relabelling (equal rows and edges per "
                                                          "rank); per aggregation only the referenced remote source "
                                                          f"rows travel, in {hp.chunks} column chunk(s), "
                                                          + ("gathered and stored into the readers' buffers over "
                                                             "NVLink by one kernel of this library, flag barriers "
                                                             "with bounded waits"
                                                             + (", pushed peer by peer on a side stream while the "
                                                                "edges of the owners that have landed are aggregated"
                                                                if hp.streamed else "")
                                                             + (", the epoch's launches replayed as one CUDA graph"
                                                                if graphed else "")
                                                             + (", later chunks pushed on a side stream beside the "
                                                                "aggregation" if getattr(args, "overlap", False) else "")
                                                             if hp.fabric is not None else
                                                             "by NCCL all-to-all"),
                                         "balanced": "degree-dealt relabelling (equal rows and edges per rank), one "
                                                     "NCCL all-gather per aggregation (source-mask rows only for "
                                                     "the backward layers)"}[mode]},
            "local_spmm_ms": round(kms.item(), 4), "exchange_ms": round(ms.item() - kms.item(), 4),
            "shards": {"edges": [int(t[0]) for t in gathered], "rows": [int(t[1]) for t in gathered],
                       "source_rows_per_aggregation": exchanged},
            "roofline": {"bound": "hbm", "kernel": "rank 0's local SpMMs of one epoch, summed",
                         "achieved": round(achieved, 1), "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "traffic": None, "algorithmic_bytes": int(algo),
                         "note": "one GPU's compulsory bytes over its local kernel time; the per-kernel roofline "
                                 "with ncu traffic is reported by the 1-GPU run of the default workload"},
            "clocks": clocks.summary(), "check": check,
            "e2e": {"value": round(e2e.item(), 4), "unit": "ms/epoch", "h2d_bytes_per_step": int(byts[0]),
                    "d2h_bytes_per_step": int(byts[1]),
                    "what": "each rank stages its rows from pinned host memory, exchanges, aggregates, copies results "
                            "back; copies in, kernels and copies out on three streams"},
            "gpu_launches": launches * args.steps, "cpu_baseline": None,
            "setup_s": round(setup_s, 2), "prep_s": round(hp.prep_s, 4),
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
