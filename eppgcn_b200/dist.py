"""Row-partitioned data parallelism for the GCN aggregation hot path.

The reference is single-GPU.  Destination rows are independent once the whole
source matrix is visible, so the graph is cut into contiguous
destination-vertex ranges with (nearly) equal edge counts, one range per rank:

  forward, per layer    local ``X_g @ W`` -> all-gather of the (narrow) post-update
                        rows into every rank's own memory -> local SpMM over the
                        rank's rows (global column ids).
  preparation           every rank marks the execution path of its own rows
                        (``mask_forward`` with ``row_offset``); the neighbour mask
                        of a step is OR-reduced over ranks before the next step.
  backward, per layer   all-gather of ``d_output`` rows -> local compacted SpMM
                        over the rank's own parts -> local ``d_input`` rows;
                        ``d_weight`` partials are all-reduced.

Remote rows always land in local memory first (NCCL over NVLink); kernels never
read a peer's memory.  The host-side logic (ranges, shards, row exchange, mask
reduction) runs unchanged on the ``gloo`` backend and is tested there.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist


def edge_balanced_ranges(indptr: np.ndarray, world: int) -> np.ndarray:
    """``world + 1`` vertex boundaries; range ``g`` is ``[b[g], b[g+1])`` and
    holds about ``E / world`` edges.  Rows are never split."""
    indptr = np.asarray(indptr, dtype=np.int64)
    n, e = indptr.shape[0] - 1, int(indptr[-1])
    targets = (np.arange(1, world, dtype=np.int64) * e) // world
    cuts = np.searchsorted(indptr, targets, side="left")
    b = np.concatenate([[0], np.clip(cuts, 0, n), [n]]).astype(np.int64)
    return np.maximum.accumulate(b)


@dataclass
class RowShard:
    """One rank's slice of the CSR: local row pointers, global column ids."""
    rank: int
    v0: int
    v1: int
    indptr: np.ndarray     # int32[v1-v0+1], starts at 0
    indices: np.ndarray    # int32[local edges], global ids

    @property
    def num_rows(self) -> int:
        return self.v1 - self.v0

    @property
    def num_edges(self) -> int:
        return int(self.indices.shape[0])


def make_shard(indptr: np.ndarray, indices: np.ndarray, bounds: np.ndarray, rank: int) -> RowShard:
    v0, v1 = int(bounds[rank]), int(bounds[rank + 1])
    e0, e1 = int(indptr[v0]), int(indptr[v1])
    local = (indptr[v0:v1 + 1].astype(np.int64) - e0).astype(np.int32)
    return RowShard(rank, v0, v1, local, np.ascontiguousarray(indices[e0:e1]))


def all_gather_rows(full: torch.Tensor, local: torch.Tensor, bounds, group=None):
    """Fills ``full[b[r]:b[r+1]]`` on every rank with rank ``r``'s ``local``
    rows.  Row counts differ between ranks, so the exchange is one broadcast
    per rank (``full`` may have a padded row stride; only ``local.size(1)``
    columns are written)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    d = local.size(1)
    v0, v1 = int(bounds[rank]), int(bounds[rank + 1])
    if local.size(0) != v1 - v0:
        raise ValueError("local rows do not match this rank's range")
    full[v0:v1, :d].copy_(local)
    if world == 1:
        return full
    ld = full.stride(0)
    if full.stride(1) != 1 or ld < full.size(1):
        raise ValueError("full must have unit column stride")
    # whole padded rows [a, b) of a range are one contiguous block of the underlying buffer
    blocks = [torch.as_strided(full, (int(bounds[r + 1]) - int(bounds[r]), ld), (ld, 1),
                               full.storage_offset() + int(bounds[r]) * ld) for r in range(world)]
    if dist.get_backend(group) == "nccl" and all(b.size(0) > 0 for b in blocks):
        # uneven all-gather: NCCL runs the per-rank broadcasts as one group, all links busy at once
        dist.all_gather(blocks, blocks[rank], group=group)
        return full
    works = [dist.broadcast(blocks[r], src=dist.get_global_rank(group, r) if group else r, group=group,
                            async_op=True) for r in range(world) if blocks[r].size(0) > 0]
    for w in works:
        w.wait()
    return full


def or_reduce_mask(mask: torch.Tensor, group=None):
    """In-place OR of a bool mask over ranks (as a byte MAX)."""
    if dist.get_world_size(group) > 1:
        as_bytes = mask.view(torch.uint8)
        dist.all_reduce(as_bytes, op=dist.ReduceOp.MAX, group=group)
    return mask


class DistHotPath:
    """One rank's device state: CSR shard, groups, prepared execution path."""

    def __init__(self, ds, dev, rank: int, world: int, back_size: int = 32, group=None):
        import eppgcn_b200
        from eppgcn_b200 import capi
        self.capi, self.dev, self.rank, self.world, self.group = capi, dev, rank, world, group
        gnna = eppgcn_b200.load_gnnadvisor()
        g = ds.graph
        self.n = g.num_nodes
        self.bounds = edge_balanced_ranges(g.indptr, world)
        sh = make_shard(g.indptr, g.indices, self.bounds, rank)
        self.shard = sh
        self.part_size = max(int(ds.avg_degree), 1)
        L = ds.num_layers
        row_cpu = torch.from_numpy(sh.indptr)
        pp, p2n = gnna.build_part(self.part_size, row_cpu)
        self.row, self.col = row_cpu.to(dev), torch.from_numpy(sh.indices).to(dev)
        self.pp, self.p2n = pp.to(dev), p2n.to(dev)
        self.deg = ds.degrees.to(dev)
        self.deg_row = self.deg[sh.v0:sh.v1]
        n_loc, e_loc = sh.num_rows, sh.num_edges
        train = ds.train_mask.to(dev)
        ngh = [torch.zeros(self.n, dtype=torch.bool, device=dev) for _ in range(L - 1)]
        edge_masks = [torch.full((e_loc,), -1, dtype=torch.int32, device=dev) for _ in range(L)]
        node_degs = [torch.zeros(n_loc, dtype=torch.int32, device=dev) for _ in range(L)]
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for i in range(L):
            src = train if i == 0 else ngh[i - 1]
            dst = ngh[i] if i < L - 1 else None
            capi.mask_forward(self.p2n, self.pp, self.col, src, dst, edge_masks[L - 1 - i], node_degs[L - 1 - i],
                              L, i + 1, row_offset=sh.v0)
            if dst is not None:
                or_reduce_mask(dst, group)
        self.path = []
        for i in range(L):
            ids, edges, valid = capi.compact_mask(edge_masks[i], self.col)
            ppb, parts = capi.split_parts(node_degs[i], e_loc, back_size)
            self.path.append(dict(id=ids, edges=edges, pp=ppb, parts=parts, valid=valid,
                                  rows=int(torch.count_nonzero(node_degs[i]).item())))
        torch.cuda.synchronize(dev)
        self.prep_s = time.perf_counter() - t0
        self.ngh_masks, self.node_degs, self.edge_masks = ngh, node_degs, edge_masks
        self.back_size = back_size

    def gather(self, full, local):
        return all_gather_rows(full, local, self.bounds, self.group)

    def forward(self, feat_full, out_local):
        return self.capi.spmm_forward(feat_full, self.row, self.col, self.deg, self.pp, self.p2n, self.part_size,
                                      out=out_local, deg_row=self.deg_row, prescaled=True)

    def backward(self, i, d_out_full, out_local):
        p = self.path[i]
        return self.capi.spmm_backward_compacted(d_out_full, p["id"], p["pp"], p["edges"], self.deg, p["parts"],
                                                 self.back_size, out=out_local, deg_row=self.deg_row,
                                                 num_rows=self.shard.num_rows)


def run_bench(args, rank: int, world: int, dev):
    """Multi-GPU arm of bench.py: the same four aggregations, row-partitioned,
    each preceded by the all-gather of its source rows.  Strong scaling: the
    graph is fixed and split over the ranks."""
    from eppgcn_b200 import graphs
    import bench as B
    dist.init_process_group("nccl", device_id=dev)
    spec = graphs.WORKLOADS[args.workload]
    if rank == 0:
        ds = graphs.load_workload(args.workload, args.seed)      # generates and caches the graph once per box
    dist.barrier()
    if rank != 0:
        ds = graphs.load_workload(args.workload, args.seed)
    n, e = ds.num_nodes, ds.num_edges
    dims = [spec["hidden"], spec["classes"]]
    hp = DistHotPath(ds, dev, rank, world, args.backsize)
    n_loc = hp.shard.num_rows
    gen = torch.Generator(device=dev).manual_seed(args.seed + rank)
    widths = (dims[0], dims[1], dims[1], dims[0])
    local_in = [torch.randn(n_loc, d, device=dev, generator=gen) for d in widths]
    full = [B.padded(n, dims[0], dev, gen), B.padded(n, dims[1], dev, gen),
            torch.empty(n, dims[1], device=dev), torch.empty(n, dims[0], device=dev)]
    outs = [torch.empty(n_loc, d, device=dev) for d in widths]

    def step():
        for k in range(4):
            hp.gather(full[k], local_in[k])
            if k < 2:
                hp.forward(full[k], outs[k])
            else:
                hp.backward(1 if k == 2 else 0, full[k], outs[k])

    stream = torch.cuda.current_stream()
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    with B.ClockSampler(dev.index) as clocks:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        dist.barrier()
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([ev0.elapsed_time(ev1) / args.steps], device=dev)
        # kernel-only share: the local SpMMs without the exchange
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(stream)
        for _ in range(args.steps):
            hp.forward(full[0], outs[0]); hp.forward(full[1], outs[1])
            hp.backward(1, full[2], outs[2]); hp.backward(0, full[3], outs[3])
        k1.record(stream)
        torch.cuda.synchronize()
        kms = torch.tensor([k0.elapsed_time(k1) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    dist.all_reduce(kms, op=dist.ReduceOp.MAX)

    # e2e: host buffers, every step stages this rank's rows in and its results out
    host_in = [torch.empty(x.shape, pin_memory=True).copy_(x) for x in local_in]
    host_out = [torch.empty(o.shape, pin_memory=True) for o in outs]

    def e2e_step():
        for k in range(4):
            local_in[k].copy_(host_in[k], non_blocking=True)
            hp.gather(full[k], local_in[k])
            (hp.forward(full[k], outs[k]) if k < 2 else hp.backward(1 if k == 2 else 0, full[k], outs[k]))
            host_out[k].copy_(outs[k], non_blocking=True)

    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    dist.barrier()
    steps2 = max(3, min(args.steps, 10))
    ev0.record(stream)
    for _ in range(steps2):
        e2e_step()
    ev1.record(stream)
    torch.cuda.synchronize()
    e2e = torch.tensor([ev0.elapsed_time(ev1) / steps2], device=dev)
    dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    byts = torch.tensor([sum(x.numel() * 4 for x in local_in), sum(o.numel() * 4 for o in outs)],
                        device=dev, dtype=torch.int64)
    dist.all_reduce(byts)
    edges = torch.tensor([hp.shard.num_edges, n_loc], device=dev, dtype=torch.int64)
    gathered = [torch.zeros_like(edges) for _ in range(world)]
    dist.all_gather(gathered, edges)
    if rank == 0:
        peak, peak_src = B.measured_peak_gbs()
        algo = B.bytes_forward(n, e, dims[0]) + B.bytes_forward(n, e, dims[1])
        line = {
            "metric": "2-layer GCN ms/epoch (fwd+bwd aggregation)", "value": round(ms.item(), 4), "unit": "ms/epoch",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms.item(), 4),
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: N={n}, E={e} directed incl. self loops, dims {dims[0]}/{dims[1]}, "
                                   f"train_ratio {spec['train_ratio']}, group size {hp.part_size}, "
                                   f"backward part size {args.backsize}",
                       "seed": args.seed, "l2": "inputs exceed L2",
                       "parallelism": f"rows{world}: destination-row ranges with equal edge counts, "
                                      f"one NCCL row all-gather per aggregation"},
            "local_spmm_ms": round(kms.item(), 4), "exchange_ms": round(ms.item() - kms.item(), 4),
            "shards": {"edges": [int(t[0]) for t in gathered], "rows": [int(t[1]) for t in gathered]},
            "roofline": {"bound": "hbm", "kernel": "all four local SpMMs", "achieved": None, "peak": peak,
                         "peak_source": peak_src, "unit": "GB/s", "frac": None, "traffic": None,
                         "note": "per-kernel roofline is reported by the 1-GPU run"},
            "clocks": clocks.summary(),
            "e2e": {"value": round(e2e.item(), 4), "unit": "ms/epoch", "h2d_bytes_per_step": int(byts[0]),
                    "d2h_bytes_per_step": int(byts[1]),
                    "what": "each rank stages its rows from pinned host memory, exchanges, aggregates, copies results back"},
            "gpu_launches": 4 * args.steps, "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
