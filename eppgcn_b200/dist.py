"""Row-partitioned data parallelism for the GCN aggregation hot path.

The reference is single-GPU.  Destination rows are independent once the whole
source matrix is visible, so every rank owns a set of destination rows.  Four
ways of choosing and exchanging them are kept, selected by ``exchange``:

  ``balanced``   (default) vertices are relabelled by a degree-sorted round robin,
                 so that every rank owns the same number of rows and (nearly) the
                 same number of edges; equal blocks make the row exchange a plain
                 ``all_gather_into_tensor``, and the backward pass gathers only the
                 rows the execution path marks (``MaskedGather``).
  ``allgather``  contiguous vertex ranges with (nearly) equal edge counts; blocks
                 are uneven, so the exchange pads to the largest one.
  ``halo``       contiguous ranges, but only the rows a rank's edges touch travel
                 (``HaloPlan``, all-to-all); slowest in practice (uneven pairs).
  ``balanced_halo``  the relabelling of ``balanced`` with a halo exchange
                 (``DealtHalo``): only the remote rows a rank's edges reference
                 travel, the rank's own rows never move, and the transfer is one
                 kernel of this package that gathers the rows and stores them
                 straight into the readers' buffers over NVLink, ordered by a flag
                 barrier with bounded waits (``PeerFabric``); NCCL all-to-all is the
                 alternative transport.  The barrier numbers itself on the device,
                 so a whole step can be captured into one CUDA graph and replayed
                 (``DistHotPath.graphed``).  ``streamed=True`` replaces push + barrier
                 + one aggregation by a push that signals every peer as its rows are
                 complete and an aggregation cut by source owner.

Per layer (``all-gather`` stands for whichever exchange the mode uses):

  forward, per layer    local ``X_g @ W`` -> all-gather of the (narrow) post-update
                        rows into every rank's own memory -> local SpMM over the
                        rank's rows (global column ids).
  preparation           every rank marks the execution path of its own rows
                        (``mask_forward`` with ``row_offset``); the neighbour mask
                        of a step is OR-reduced over ranks before the next step.
  backward, per layer   all-gather of ``d_output`` rows -> local compacted SpMM
                        over the rank's own parts -> local ``d_input`` rows;
                        ``d_weight`` partials are all-reduced.

Remote rows always land in the reader's own memory before any kernel reads them
(NCCL, or peer stores by the owner); no kernel loads from a peer's memory.  The
host-side logic (ranges, shards, row exchange, mask
reduction) runs unchanged on the ``gloo`` backend and is tested there.
"""
from __future__ import annotations

import json
import os
import contextlib
import time
from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist


def _sync(dev):
    """Host wait for the device's queued work; nothing to wait for on the CPU (gloo tests)."""
    if torch.device(dev).type == "cuda":
        torch.cuda.synchronize(dev)


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


def balanced_relabel(indptr: np.ndarray, world: int):
    """Vertex relabelling that gives every rank the same number of rows AND
    about the same number of edges: vertices sorted by degree are dealt to the
    ranks round-robin; rank ``g`` owns new ids ``[g*n_loc, (g+1)*n_loc)``.

    Equal row counts let the row exchange be one plain NCCL all-gather (2.3x
    faster here than the grouped broadcasts uneven blocks need), and dealing
    the hubs out evens the local work.  Returns ``(new_of_old[N], n_loc)``;
    new ids ``>= N`` up to ``world*n_loc`` are padding rows without edges.
    """
    deg = np.diff(np.asarray(indptr, dtype=np.int64))
    n = deg.shape[0]
    n_loc = -(-n // world)
    order = np.argsort(-deg, kind="stable")
    i = np.arange(n, dtype=np.int64)
    new_of_old = np.empty(n, dtype=np.int64)
    new_of_old[order] = (i % world) * n_loc + i // world
    return new_of_old, n_loc


def make_relabelled_shard(indptr: np.ndarray, indices: np.ndarray, new_of_old: np.ndarray, n_loc: int,
                          rank: int, world: int) -> RowShard:
    """Rank ``rank``'s rows of the relabelled graph: local row pointers, column
    ids in the new numbering (rows keep their edges' original order)."""
    n = indptr.shape[0] - 1
    old_of_new = np.full(n_loc * world, -1, dtype=np.int64)
    old_of_new[new_of_old] = np.arange(n, dtype=np.int64)
    mine = old_of_new[rank * n_loc:(rank + 1) * n_loc]
    valid = mine >= 0
    safe = np.where(valid, mine, 0)
    lens = np.where(valid, indptr[safe + 1].astype(np.int64) - indptr[safe], 0)
    local = np.zeros(n_loc + 1, dtype=np.int64)
    np.cumsum(lens, out=local[1:])
    starts = np.repeat(indptr[safe].astype(np.int64) - local[:-1], lens)
    src = starts + np.arange(int(local[-1]), dtype=np.int64)
    cols = new_of_old[indices[src]].astype(np.int32)
    return RowShard(rank, rank * n_loc, (rank + 1) * n_loc, local.astype(np.int32), cols)


def balanced_shard_device(indptr: torch.Tensor, indices: torch.Tensor, rank: int, world: int):
    """Torch twin of :func:`balanced_relabel` + :func:`make_relabelled_shard`
    for graphs that already live on a device.  Returns ``(new_of_old int64[N],
    n_loc, local_indptr int32[n_loc+1], cols int32[local edges])``."""
    dev = indptr.device
    deg = (indptr[1:] - indptr[:-1]).long()
    n = deg.numel()
    n_loc = -(-n // world)
    order = torch.sort(deg, descending=True, stable=True).indices
    i = torch.arange(n, device=dev)
    new_of_old = torch.empty(n, dtype=torch.int64, device=dev)
    new_of_old[order] = (i % world) * n_loc + i // world
    mine = order[rank::world]                       # old ids of this rank's rows, in local row order
    lens = torch.zeros(n_loc, dtype=torch.int64, device=dev)
    lens[:mine.numel()] = deg[mine]
    local = torch.zeros(n_loc + 1, dtype=torch.int64, device=dev)
    torch.cumsum(lens, 0, out=local[1:])
    first = indptr[mine].long() - local[:mine.numel()]
    src = torch.repeat_interleave(first, lens[:mine.numel()]) + torch.arange(int(local[-1]), device=dev)
    cols = new_of_old[indices[src].long()].to(torch.int32)
    return new_of_old, n_loc, local.to(torch.int32), cols


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
    if world == 1:
        full[v0:v1, :d].copy_(local)
        return full
    ld = full.stride(0)
    if full.stride(1) != 1 or ld < full.size(1):
        raise ValueError("full must have unit column stride")
    # whole padded rows [a, b) of a range are one contiguous block of the underlying buffer
    blocks = [torch.as_strided(full, (int(bounds[r + 1]) - int(bounds[r]), ld), (ld, 1),
                               full.storage_offset() + int(bounds[r]) * ld) for r in range(world)]
    if all(b.size(0) == blocks[0].size(0) for b in blocks) and full.size(0) == world * blocks[0].size(0) \
            and dist.get_backend(group) == "nccl":
        # equal blocks: one plain all-gather over the whole padded buffer
        whole = torch.as_strided(full, (full.size(0), ld), (ld, 1), full.storage_offset())
        mine = _padded_rows(local)
        if mine.size(1) != ld or not mine.is_contiguous():      # different padding: go through the own block
            full[v0:v1, :d].copy_(local)
            mine = blocks[rank]
        dist.all_gather_into_tensor(whole, mine, group=group)
        return full
    full[v0:v1, :d].copy_(local)
    if dist.get_backend(group) == "nccl" and all(b.size(0) > 0 for b in blocks):
        # uneven all-gather: NCCL runs the per-rank broadcasts as one group, all links busy at once
        dist.all_gather(blocks, blocks[rank], group=group)
        return full
    works = [dist.broadcast(blocks[r], src=dist.get_global_rank(group, r) if group else r, group=group,
                            async_op=True) for r in range(world) if blocks[r].size(0) > 0]
    for w in works:
        w.wait()
    return full


def check_agreement(values: dict, group=None, device=None):
    """Raises on EVERY rank when the ranks do not hold the same integers: ``values`` maps a name
    (the same names in the same order on all ranks) to an int.  Used before the first exchange, so
    that a rank started with another graph, seed, layer count or partition fails with a message
    that names the field instead of exchanging rows of the wrong shape.  One all-gather of a few
    64-bit words."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    names = list(values)
    mine = torch.tensor([int(values[k]) for k in names], dtype=torch.int64, device=device)
    world = dist.get_world_size(group)
    got = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(got, mine, group=group)
    table = torch.stack(got).cpu()
    for j, name in enumerate(names):
        col = table[:, j]
        if not bool((col == col[0]).all()):
            raise RuntimeError(f"the ranks disagree on {name}: " +
                               ", ".join(f"rank {r}: {int(v)}" for r, v in enumerate(col.tolist())))


def or_reduce_mask(mask: torch.Tensor, group=None):
    """In-place OR of a bool mask over ranks (as a byte MAX)."""
    if dist.get_world_size(group) > 1:
        as_bytes = mask.view(torch.uint8)
        dist.all_reduce(as_bytes, op=dist.ReduceOp.MAX, group=group)
    return mask


def _padded_rows(t: torch.Tensor) -> torch.Tensor:
    """The whole rows (row stride wide) behind a ``[n, d]`` view with unit column stride."""
    if t.dim() != 2 or (t.size(1) > 1 and t.stride(1) != 1):
        raise ValueError("expected a 2-D tensor with unit column stride")
    ld = t.stride(0) if t.size(0) > 1 else max(t.stride(0), t.size(1))
    return t if ld == t.size(1) else torch.as_strided(t, (t.size(0), ld), (ld, 1), t.storage_offset())


class HaloPlan:
    """Exchange of only the source rows a rank's edges reference.

    ``cols`` holds global source ids (one per edge).  The distinct ids, sorted,
    define the rank's compact source buffer; because every owner's range is a
    contiguous id interval, that order is also "grouped by owner", so one
    all-to-all with per-owner row counts fills the buffer in place.  ``remap``
    gives every edge its position in the buffer and replaces the global column
    ids in the kernels' arguments.  Built once per aggregation (forward: all
    local edges; backward of a layer: the compacted edges of its path).
    """

    def __init__(self, cols: torch.Tensor, bounds, rank: int, world: int, group=None):
        dev = cols.device
        self.rank, self.world, self.group = rank, world, group
        ids = cols.long()
        self.needed = torch.unique(ids)                                    # sorted global ids
        self.remap = torch.searchsorted(self.needed, ids).to(torch.int32)
        b = torch.as_tensor(np.asarray(bounds, dtype=np.int64), device=dev)
        cut = torch.searchsorted(self.needed, b)                           # owner r: needed[cut[r]:cut[r+1]]
        self.recv_counts = (cut[1:] - cut[:-1]).tolist()
        owner = torch.bucketize(self.needed, b[1:], right=True)
        request = self.needed - b[owner]                                   # row ids local to their owner
        counts_in = torch.tensor(self.recv_counts, dtype=torch.int64, device=dev)
        counts_out = torch.empty_like(counts_in)
        if world > 1:
            dist.all_to_all_single(counts_out, counts_in, group=group)
        else:
            counts_out.copy_(counts_in)
        self.send_counts = counts_out.tolist()
        self.send_idx = torch.empty(int(sum(self.send_counts)), dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_to_all_single(self.send_idx, request, self.send_counts, self.recv_counts, group=group)
        else:
            self.send_idx.copy_(request)
        self.num_rows = int(self.needed.numel())

    def exchange(self, local: torch.Tensor) -> torch.Tensor:
        """``local``: this rank's rows ``[n_local, d]`` (row stride may be
        padded).  Returns the compact source buffer ``[num_rows, d]`` with the
        same row stride, row ``k`` holding global row ``needed[k]``."""
        rows = _padded_rows(local)
        send = rows.index_select(0, self.send_idx)
        if self.world == 1:
            return send[:, :local.size(1)]
        buf = torch.empty(self.num_rows, rows.size(1), dtype=local.dtype, device=local.device)
        dist.all_to_all_single(buf, send, self.recv_counts, self.send_counts, group=self.group)
        return buf[:, :local.size(1)]


class PeerFabric:
    """Peer-mapped buffers of the ranks of one node and a flag barrier over them.

    Buffers come from torch's symmetric-memory allocator, which maps every
    rank's copy into every process; only this package's own kernels
    (``eppgcn_push_rows``, ``eppgcn_peer_barrier``) ever touch a peer's copy --
    plain stores and flag words, no library kernel is handed a peer address.
    Every barrier wait is bounded; :meth:`check` raises if one ran out."""

    def __init__(self, dev, rank: int, world: int, group=None, max_polls: int = 10_000_000):
        import torch.distributed._symmetric_memory as symm
        from eppgcn_b200 import capi
        self.symm, self.capi = symm, capi
        self.dev, self.rank, self.world = dev, rank, world
        self.group = group if group is not None else dist.group.WORLD
        self._keep = []
        flags, self.flag_ptrs = self.alloc((64,), torch.int32)
        flags.zero_()
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        # Barriers are numbered by a word on the device (every launch takes the next number), so that a captured
        # sequence of launches can be replayed; ``count`` is the host's tally of the barriers it has enqueued.
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.count, self.max_polls = 0, max_polls    # a poll takes about a microsecond: ranks may be ~10 s apart
        # The streamed exchange: word r of ``landed`` is stored by rank r when its rows of the current exchange
        # have arrived here; ``epoch`` numbers the exchanges (advanced on the device, in stream order);
        # ``done`` is the push kernel's scratch; pushes run on ``comm`` beside the aggregation.
        self.landed, self.landed_ptrs = self.alloc((64,), torch.int32)
        self.landed.zero_()
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(16, dtype=torch.int32, device=dev)
        self.comm = torch.cuda.Stream(device=dev, priority=-1)     # its blocks are placed before the aggregation's
        _sync(dev)
        dist.barrier(self.group)                     # every rank's flag words are zero before the first barrier

    @staticmethod
    def available(dev, group=None) -> bool:
        """Peer stores need CUDA devices of one node under an NCCL group."""
        return torch.device(dev).type == "cuda" and dist.get_backend(group) == "nccl"

    def alloc(self, shape, dtype=torch.float32):
        """A buffer of the same shape on every rank; returns ``(own tensor, [address of rank r's copy])``."""
        t = self.symm.empty(tuple(shape), dtype=dtype, device=self.dev)
        hdl = self.symm.rendezvous(t, self.group)
        peers = [hdl.get_buffer(r, tuple(shape), dtype) for r in range(self.world)]
        self._keep.append((t, hdl, peers))
        return t, [p.data_ptr() for p in peers]

    def barrier(self):
        self.count += 1
        self.capi.peer_barrier_counted(self.flag_ptrs, self.rank, self.counter, self.status, self.max_polls)

    @contextlib.contextmanager
    def side_stream(self):
        """Work enqueued inside runs on the fabric's side stream, after everything the current stream holds
        so far; :meth:`join_side_stream` makes the current stream wait for it."""
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream())
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(ready)
            yield
            self._side_done = torch.cuda.Event()
            self._side_done.record(self.comm)

    def join_side_stream(self):
        torch.cuda.current_stream().wait_event(self._side_done)

    def check(self):
        code = int(self.status.item())
        if code != 0:
            raise RuntimeError(f"a bounded wait for another GPU ran out (status {code}): a rank is late or gone")


class _Landed:
    """What :meth:`DealtHalo.start` hands out per chunk on the push transport:
    ``wait()`` makes the current stream wait for this rank's push of the chunk
    (when it ran on the side stream) and then for every rank's, through a
    barrier.  All ranks wait for the chunks in the same order."""

    def __init__(self, fabric, event=None):
        self.fabric, self.event = fabric, event

    def wait(self):
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)
        self.fabric.barrier()


class DealtHalo:
    """Halo exchange over equal row blocks (the dealt-out relabelling), with the
    rank's own rows kept out of the all-to-all and the transfer cut into column
    chunks so that the aggregation of one chunk runs while the next one travels.

    The source buffer of chunk ``c`` is ``[num_remote + n_loc, d / chunks]``:
    first the remote rows this rank's edges reference, sorted by global id (hence
    grouped by owner), then the rank's own ``n_loc`` rows.  ``remap`` gives every
    edge its row in that buffer; ``order`` lists the global ids in buffer order.
    """

    def __init__(self, cols: torch.Tensor, n_loc: int, rank: int, world: int, group=None, fabric=None):
        dev = cols.device
        self.rank, self.world, self.group, self.n_loc = rank, world, group, n_loc
        self.fabric = fabric if world > 1 else None
        self.overlap, self._side = False, None       # push chunk c+1 on a side stream beside the aggregation of chunk c
        self.lead_barrier = False                    # True: always wait for the readers before a push (see start)
        ids = cols.long()
        v0 = rank * n_loc
        own = (ids >= v0) & (ids < v0 + n_loc)
        remote_ids = ids[~own]
        self.needed = torch.unique(remote_ids)                             # sorted global ids of other ranks' rows
        r = int(self.needed.numel())
        remap = torch.empty_like(ids)
        remap[~own] = torch.searchsorted(self.needed, remote_ids)
        remap[own] = ids[own] - v0 + r
        self.remap = remap.to(torch.int32)
        b = torch.arange(world + 1, device=dev, dtype=torch.int64) * n_loc
        cut = torch.searchsorted(self.needed, b)
        self.cut = cut                                 # buffer rows [cut[o], cut[o+1]) come from rank o
        counts_in = cut[1:] - cut[:-1]
        self.recv_counts = counts_in.tolist()
        request = self.needed % n_loc                                      # row ids local to their owner
        counts_out = torch.empty_like(counts_in)
        if world > 1:
            dist.all_to_all_single(counts_out, counts_in, group=group)
        else:
            counts_out.copy_(counts_in)
        self.send_counts = counts_out.tolist()
        self.send_idx = torch.empty(int(sum(self.send_counts)), dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_to_all_single(self.send_idx, request, self.send_counts, self.recv_counts, group=group)
        self.num_remote, self.num_rows = r, r + n_loc
        self.order = torch.cat([self.needed, torch.arange(v0, v0 + n_loc, device=dev)])
        self._bufs, self._stamps = {}, {}
        if self.fabric is not None:
            # peer stores: where this rank's rows start in every reader's buffer, and one buffer size for all ranks
            first_in = cut[:-1].clone()
            first_out = torch.empty_like(first_in)
            dist.all_to_all_single(first_out, first_in, group=group)
            self.peer_first_row = first_out.tolist()
            self.send_ptr = [0] + np.cumsum(self.send_counts).tolist()
            # every rank starts with its right-hand neighbour's rows, so no peer is everybody's first target
            self.push_start = self.send_ptr[(rank + 1) % world] % max(self.send_ptr[-1], 1)
            self.send_idx32 = self.send_idx.to(torch.int32)
            rows_max = torch.tensor([self.num_rows], device=dev, dtype=torch.int64)
            dist.all_reduce(rows_max, op=dist.ReduceOp.MAX, group=group)
            self.rows_max = int(rows_max.item())

    def buffers(self, d: int, chunks: int):
        """Per-chunk (send rows, source buffer) pairs for a ``d``-wide matrix; the
        chunk count falls back to 1 when ``d`` does not split into 16-byte aligned rows."""
        if chunks < 1 or d % (4 * chunks):
            chunks = 1
        key = (d, chunks)
        if key not in self._bufs:
            dc = d // chunks
            dev = self.send_idx.device
            if self.fabric is not None:
                ld = (dc + 3) // 4 * 4               # rows travel as whole 16-byte pieces; padding stays zero
                made = []
                for _ in range(chunks):
                    whole, peers = self.fabric.alloc((self.rows_max, ld))
                    whole.zero_()
                    made.append((peers, whole[:self.num_rows, :dc]))
                self._bufs[key] = made
            else:
                self._bufs[key] = [(torch.empty(self.send_idx.numel(), dc, device=dev),
                                    torch.zeros(self.num_rows, dc, device=dev)) for _ in range(chunks)]
        return self._bufs[key]

    def own_rows(self, d: int, chunks: int = 1):
        """The places of the rank's own rows inside the source buffers, one
        ``[n_loc, d / chunks]`` view per chunk.  A producer that writes its rows
        there (column block by column block) saves the copy :meth:`start` makes."""
        return [buf[self.num_remote:] for _, buf in self.buffers(d, chunks)]

    def _place_own(self, buf, rows, scale):
        """This rank's rows into their place in a source buffer; with ``scale`` (its own
        vertices' source-side factors) they are multiplied on the way, so that every
        rank's edges find pre-scaled rows."""
        if scale is None:
            buf[self.num_remote:].copy_(rows)
        else:
            from eppgcn_b200 import capi
            capi.pack_scaled_rows(rows, scale, None, out=buf[self.num_remote:])

    def start(self, local, chunks: int = 1, d: int = 0, scale=None):
        """Enqueues the exchange of ``local [n_loc, d]``, one all-to-all per column
        chunk; ``local = None``: the rows already sit in :meth:`own_rows` (``d``
        names the width).  ``scale [n_loc]``: the rows are multiplied by it while they
        are copied into place (not with ``local = None``).  Returns ``[(work, buffer)]``;
        ``work.wait()`` makes the current stream wait for that chunk only."""
        d = local.size(1) if local is not None else d
        out = []
        bufs = self.buffers(d, chunks)
        if self.fabric is not None and isinstance(bufs[0][0], list):
            # Peer stores: wait until no rank reads these buffers any more, push, wait until every push has
            # landed.  The first wait is only needed when no barrier has passed since these buffers were last
            # aggregated from: a rank arrives at any later barrier after that aggregation (same stream), so
            # whoever has left such a barrier may overwrite them.  An epoch that alternates between buffers
            # (layers of different width, forward and backward) therefore pays one barrier per aggregation.
            key = (d, len(bufs))
            stamp = self._stamps.get(key)
            if self.lead_barrier or stamp is None or self.fabric.count <= stamp or (self.overlap and len(bufs) > 1):
                self.fabric.barrier()
            if local is not None:
                for c, (_, buf) in enumerate(bufs):
                    dc = buf.size(1)
                    self._place_own(buf, local[:, c * dc:(c + 1) * dc], scale)

            def push(peers, buf):
                wide = _padded_rows(buf[self.num_remote:])
                self.fabric.capi.push_rows(wide, self.send_idx32, self.send_ptr, peers, self.peer_first_row,
                                           wide.size(1), start_row=self.push_start)

            if not (self.overlap and len(bufs) > 1):
                for peers, buf in bufs:
                    push(peers, buf)
                    out.append((None, buf))
                self.fabric.barrier()
                self._stamps[key] = self.fabric.count
                return out
            # chunk 0 on this stream; the later chunks on a side stream, each behind the one before it, so that
            # they travel while the caller aggregates the chunks that have landed
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream(device=bufs[0][1].device)
            push(*bufs[0])
            out.append((_Landed(self.fabric), bufs[0][1]))
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(self._side):
                self._side.wait_event(ready)
                for peers, buf in bufs[1:]:
                    push(peers, buf)
                    done = torch.cuda.Event()
                    done.record(self._side)
                    out.append((_Landed(self.fabric, done), buf))
            return out
        for c, (send, buf) in enumerate(bufs):
            dc = send.size(1)
            if local is not None:
                self._place_own(buf, local[:, c * dc:(c + 1) * dc], scale)
            part = buf[self.num_remote:]
            work = None
            if self.world > 1:                   # every rank joins, also one that neither sends nor receives
                torch.index_select(part, 0, self.send_idx, out=send)
                work = dist.all_to_all_single(buf[:self.num_remote], send, self.recv_counts, self.send_counts,
                                              group=self.group, async_op=True)
            out.append((work, buf))
        return out


    def needs_barrier(self, key) -> bool:
        """Whether an exchange into the buffers ``key`` must first wait for their readers: only when no
        barrier has been enqueued since they were last aggregated from (see :meth:`start`)."""
        stamp = self._stamps.get(key)
        return self.lead_barrier or stamp is None or self.fabric.count <= stamp

    def start_streamed(self, local, buf, peers, scale=None):
        """The streamed form of the peer-store exchange of one buffer: the rows are pushed peer by peer on
        the fabric's side stream, every peer being told as soon as its rows are complete, while the caller
        aggregates on the current stream (first the edges whose sources it owns, then owner by owner,
        each launch behind a wait for that owner's word), and calls :meth:`end_streamed` after its last
        aggregation launch."""
        fab = self.fabric
        key = (buf.size(1), "streamed", buf.data_ptr())
        fab.capi.bump_counter(fab.epoch)
        if self.needs_barrier(key):
            fab.barrier()
        if local is not None:
            self._place_own(buf, local, scale)
        with fab.side_stream():
            wide = _padded_rows(buf[self.num_remote:])
            fab.capi.push_rows_signal(wide, self.send_idx32, self.send_ptr, peers, self.peer_first_row, wide.size(1),
                                      self.rank, fab.landed_ptrs, fab.epoch, fab.done)
        self._last_key = key

    def end_streamed(self):
        """After the caller's last aggregation launch of a streamed exchange: the current stream waits for
        the end of this rank's push, and the buffer counts as read up to here."""
        self.fabric.join_side_stream()
        self._stamps[self._last_key] = self.fabric.count


class MaskedGather:
    """Exchange of the rows selected by a vertex mask that every rank holds
    (the source mask of a backward layer: only those rows of ``d_output`` are
    ever read).  For equal row blocks per rank.  Rank ``g``'s selected rows are
    packed into ``cap`` slots (the largest per-rank count), so the exchange is
    one plain all-gather of ``world * cap`` rows; ``pos`` maps a vertex id to
    its slot and replaces the column ids in the kernel's arguments."""

    def __init__(self, mask: torch.Tensor, n_loc: int, rank: int, world: int, group=None):
        self.rank, self.world, self.group = rank, world, group
        blocks = mask.view(world, n_loc)
        counts = blocks.sum(1)
        self.cap = max(int(counts.max().item()), 1)
        within = torch.cumsum(blocks, 1, dtype=torch.int64) - 1
        slot = torch.arange(world, device=mask.device, dtype=torch.int64)[:, None] * self.cap + within
        self.pos = torch.where(blocks, slot, torch.zeros_like(slot)).view(-1).to(torch.int32)
        self.send_idx = torch.nonzero(blocks[rank]).view(-1)
        self.count = int(self.send_idx.numel())
        self.num_rows = world * self.cap
        self.selected = torch.nonzero(mask).view(-1)            # vertex ids, in slot order per rank

    def compact(self, per_vertex: torch.Tensor, fill=0) -> torch.Tensor:
        """A per-vertex array rearranged into slot order."""
        out = torch.full((self.num_rows,), fill, dtype=per_vertex.dtype, device=per_vertex.device)
        out[self.pos[self.selected].long()] = per_vertex[self.selected]
        return out

    def exchange(self, local: torch.Tensor) -> torch.Tensor:
        rows = _padded_rows(local)
        send = torch.empty(self.cap, rows.size(1), dtype=local.dtype, device=local.device)
        if self.count:
            torch.index_select(rows, 0, self.send_idx, out=send[:self.count])
        if self.world == 1:
            return send[:, :local.size(1)]
        buf = torch.empty(self.num_rows, rows.size(1), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(buf, send, group=self.group)
        return buf[:, :local.size(1)]


class DistHotPath:
    """One rank's device state: CSR shard, groups, prepared execution path and
    the exchange plans.  ``exchange``:

    ``"balanced"``   (default) vertices relabelled so that every rank owns the same
                     number of rows and about the same number of edges; the row
                     exchange is one plain NCCL all-gather.
    ``"allgather"``  contiguous id ranges with equal edge counts, uneven blocks
                     (grouped broadcasts).
    ``"halo"``       same ranges, only referenced rows travel (all-to-all); least
                     bytes, but NCCL send/recv was the slowest of the three on
                     8 x B200 for this graph.
    ``"balanced_halo"``  the relabelling of ``balanced`` with the exchange of
                     ``halo``: the dealt-out rows make the per-pair row counts of
                     the all-to-all nearly equal, and only referenced rows travel.
    """

    def __init__(self, ds, dev, rank: int, world: int, back_size: int = 32, group=None,
                 exchange: str = "balanced", chunks: int = 1, transport: str = "push", overlap: bool = False,
                 streamed: bool = False, owner_groups: int = 0):
        import eppgcn_b200
        from eppgcn_b200 import capi
        self.capi, self.dev, self.rank, self.world, self.group = capi, dev, rank, world, group
        self.mode, self.chunks, self.fabric, self.streamed = exchange, chunks, None, False
        gnna = eppgcn_b200.load_gnnadvisor()
        on_device = torch.is_tensor(getattr(ds, "indptr", None))      # DeviceWorkload: the graph never touches the host
        relabel = exchange in ("balanced", "balanced_halo")
        halo = exchange in ("halo", "balanced_halo")
        if on_device:
            if not relabel:
                raise ValueError("device-resident workloads support the balanced and balanced_halo modes")
            new_of_old, n_loc, local_ptr, cols = balanced_shard_device(ds.indptr, ds.indices, rank, world)
            self.new_of_old = new_of_old
            self.n = n_loc * world
            self.bounds = np.arange(world + 1, dtype=np.int64) * n_loc
            sh = RowShard(rank, rank * n_loc, (rank + 1) * n_loc, local_ptr.cpu(), cols)
            deg_t = torch.ones(self.n, device=dev)
            deg_t[new_of_old] = ds.degrees.to(dev)
            train_t = torch.zeros(self.n, dtype=torch.bool, device=dev)
            train_t[new_of_old] = ds.train_mask.to(dev)
            del new_of_old
        elif relabel:
            # relabelled graph: equal rows per rank, hubs dealt out; every per-vertex array follows the new ids
            g = ds.graph
            degrees_np, train_np = ds.degrees.cpu().numpy(), ds.train_mask.cpu().numpy()
            self.new_of_old, n_loc = balanced_relabel(g.indptr, world)
            self.n = n_loc * world
            self.bounds = np.arange(world + 1, dtype=np.int64) * n_loc
            sh = make_relabelled_shard(g.indptr, g.indices, self.new_of_old, n_loc, rank, world)
            deg_new = np.ones(self.n, dtype=np.float32)
            deg_new[self.new_of_old] = degrees_np
            train_new = np.zeros(self.n, dtype=bool)
            train_new[self.new_of_old] = train_np
            degrees_np, train_np = deg_new, train_new
        else:
            g = ds.graph
            degrees_np, train_np = ds.degrees.cpu().numpy(), ds.train_mask.cpu().numpy()
            self.new_of_old = None
            self.n = g.num_nodes
            self.bounds = edge_balanced_ranges(g.indptr, world)
            sh = make_shard(g.indptr, g.indices, self.bounds, rank)
        self.shard = sh
        self.part_size = max(int(ds.avg_degree), 1)
        L = ds.num_layers
        # every rank must have cut the same graph the same way before a single row is exchanged
        check_agreement({"the vertex count": self.n, "the edge count": int(ds.num_edges), "the layer count": L,
                         "the backward part size": back_size, "the column chunk count": chunks,
                         "the first partition boundary": int(self.bounds[1]),
                         "the train-mask size": int(ds.train_mask.sum().item() if torch.is_tensor(ds.train_mask)
                                                    else np.asarray(ds.train_mask).sum())},
                        group, dev if torch.device(dev).type == "cuda" else None)
        row_cpu = sh.indptr if on_device else torch.from_numpy(sh.indptr)
        if on_device:         # the graph never left the GPU: its groups are built there too
            pp, p2n = capi.build_part_device(self.part_size, local_ptr, sh.num_edges)
        else:
            pp, p2n = gnna.build_part(self.part_size, row_cpu)
        self.row = row_cpu.to(dev)
        self.col = sh.indices if on_device else torch.from_numpy(sh.indices).to(dev)
        self.pp, self.p2n = pp.to(dev), p2n.to(dev)
        self.deg = deg_t if on_device else torch.from_numpy(degrees_np).to(dev)
        self.deg_row = self.deg[sh.v0:sh.v1]
        n_loc, e_loc = sh.num_rows, sh.num_edges
        self.n_loc = n_loc
        train = train_t if on_device else torch.from_numpy(train_np).to(dev)
        ngh = [torch.zeros(self.n, dtype=torch.bool, device=dev) for _ in range(L - 1)]
        edge_masks = [torch.full((e_loc,), -1, dtype=torch.int32, device=dev) for _ in range(L)]
        node_degs = [torch.zeros(n_loc, dtype=torch.int32, device=dev) for _ in range(L)]
        _sync(dev)
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
        _sync(dev)
        self.prep_s = time.perf_counter() - t0
        self.ngh_masks, self.node_degs, self.edge_masks = ngh, node_degs, edge_masks
        self.back_size = back_size
        if exchange == "balanced":
            # a backward layer reads d_output only on its step's source mask: exchange just those rows
            t0 = time.perf_counter()
            for j, p in enumerate(self.path):
                step = L - 1 - j
                src = train if step == 0 else ngh[step - 1]
                plan = MaskedGather(src, n_loc, rank, world, group)
                edges_c = torch.zeros_like(p["edges"])
                edges_c[:p["valid"]] = plan.pos[p["edges"][:p["valid"]].long()]
                p.update(plan=plan, edges_c=edges_c, deg_c=plan.compact(self.deg, 0.0))
            _sync(dev)
            self.plan_s = time.perf_counter() - t0
        if exchange == "balanced_halo":
            t0 = time.perf_counter()
            if transport not in ("push", "nccl"):
                raise ValueError("transport must be 'push' (peer stores by this package's kernels) or 'nccl'")
            if transport == "push" and world > 1 and PeerFabric.available(dev, group):
                # peer-mapped buffers may be unavailable (no peer access between the devices, allocator support
                # missing): every rank must then agree to use the NCCL all-to-all instead
                try:
                    self.fabric, why = PeerFabric(dev, rank, world, group), ""
                except Exception as exc:           # noqa: BLE001 - any failure means "no peer stores here"
                    self.fabric, why = None, repr(exc)
                agreed = torch.tensor([0 if self.fabric is None else 1], device=dev)
                dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
                if int(agreed.item()) == 0:
                    if rank == 0:
                        import sys
                        print("eppgcn_b200.dist: peer-store transport unavailable, using NCCL all-to-all"
                              + (f" ({why[:200]})" if why else ""), file=sys.stderr, flush=True)
                    self.fabric = None
            # streamed: push and aggregation overlap owner by owner (peer-store transport, no chunk overlap)
            self.streamed = streamed and self.fabric is not None and not overlap
            self.owner_groups = owner_groups if owner_groups > 0 else world
            self.fwd_plan = DealtHalo(self.col, n_loc, rank, world, group, self.fabric)
            self.fwd_plan.overlap = overlap
            self.col_c = self.fwd_plan.remap
            for p in self.path:
                plan = DealtHalo(p["edges"][:p["valid"]], n_loc, rank, world, group, self.fabric)
                plan.overlap = overlap
                edges_c = torch.zeros_like(p["edges"])
                edges_c[:p["valid"]] = plan.remap
                p.update(plan=plan, edges_c=edges_c, deg_c=self.deg[plan.order].contiguous())
            _sync(dev)
            self.plan_s = time.perf_counter() - t0
        elif halo:
            t0 = time.perf_counter()
            self.fwd_plan = HaloPlan(self.col, self.bounds, rank, world, group)
            self.col_c = self.fwd_plan.remap
            for p in self.path:
                plan = HaloPlan(p["edges"][:p["valid"]], self.bounds, rank, world, group)
                edges_c = torch.zeros_like(p["edges"])
                edges_c[:p["valid"]] = plan.remap
                p.update(plan=plan, edges_c=edges_c, deg_c=self.deg[plan.needed].contiguous())
            _sync(dev)
            self.plan_s = time.perf_counter() - t0

    def gather(self, full, local):
        return all_gather_rows(full, local, self.bounds, self.group)

    def _tile_plan(self, which: str, num_sources: int):
        """The tiled-kernel plan of this rank's forward edge list, made at first use: ``"full"`` over
        the global column ids, ``"halo"`` over positions in the exchange buffer."""
        plans = self.__dict__.setdefault("_fwd_tile_plans", {})
        if which not in plans:
            col = self.col if which == "full" else self.col_c
            plans[which] = self.capi.TilePlan.from_csr(self.row, col, num_sources=num_sources)
        return plans[which]

    @staticmethod
    def _tiles_can_read(buf) -> bool:
        return buf.stride(0) % 4 == 0 and buf.data_ptr() % 16 == 0

    def forward(self, feat_full, out_local):
        """Local forward aggregation over a whole-graph source matrix (pre-scaled rows)."""
        if self._tiles_can_read(feat_full):
            return self.capi.spmm_tiles(feat_full, self._tile_plan("full", self.n), self.deg_row, out=out_local)
        return self.capi.spmm_forward(feat_full, self.row, self.col, self.deg, self.pp, self.p2n, self.part_size,
                                      out=out_local, deg_row=self.deg_row, prescaled=True)

    def backward(self, i, d_out_full, out_local):
        p = self.path[i]
        return self.capi.spmm_backward_compacted(d_out_full, p["id"], p["pp"], p["edges"], self.deg, p["parts"],
                                                 self.back_size, out=out_local, deg_row=self.deg_row,
                                                 num_rows=self.shard.num_rows)

    def _halo_spmm(self, kind, i, buf, out):
        if kind == "fwd":
            if self._tiles_can_read(buf):
                return self.capi.spmm_tiles(buf, self._tile_plan("halo", self.fwd_plan.num_rows), self.deg_row,
                                            out=out)
            return self.capi.spmm_forward(buf, self.row, self.col_c, self.deg, self.pp, self.p2n, self.part_size,
                                          out=out, deg_row=self.deg_row, prescaled=True)
        p = self.path[i]
        if p.get("prescaled", {}).get(buf.size(1)):
            # the exchange already multiplied every row by its source-side factor (see _dealt_op)
            if "tile_plan" not in p:
                p["tile_plan"] = self.capi.TilePlan.from_ids(p["id"], p["edges_c"], p["valid"], self.shard.num_rows,
                                                             num_sources=p["plan"].num_rows)
            return self.capi.spmm_tiles(buf, p["tile_plan"], self.deg_row, out=out)
        return self.capi.spmm_backward_compacted(buf, p["id"], p["pp"], p["edges_c"], p["deg_c"], p["parts"],
                                                 self.back_size, out=out, deg_row=self.deg_row,
                                                 num_rows=self.shard.num_rows)

    def _segment_plans(self, kind, i):
        """The edge list of one aggregation cut by the owner of the source row into tile plans:
        ``[(owners, plan)]``, first the edges whose sources this rank owns (``owners = ()``), then the other
        ranks in the order their rows arrive (rank+1, rank+2, ...), bundled into at most
        ``self.owner_groups`` groups of consecutive owners.  Sources are positions in the exchange buffer;
        a plan is ``None`` when the rank's own part has no edge."""
        cache = self.__dict__.setdefault("_seg_plans", {})
        i = 0 if kind == "fwd" else i                   # every forward layer aggregates over the same edge list
        if (kind, i) in cache:
            return cache[(kind, i)]
        dev, n_loc, w = self.dev, self.n_loc, self.world
        if kind == "fwd":
            plan = self.fwd_plan
            pos = self.col_c.long()
            counts = (self.row[1:] - self.row[:-1]).long()
            rows = torch.repeat_interleave(torch.arange(n_loc, device=dev), counts)
        else:
            p = self.path[i]
            plan = p["plan"]
            pos = p["edges_c"][:p["valid"]].long()
            rows = p["id"][:p["valid"]].long()
        # positions from cut[o] up to cut[o+1] belong to owner o; the rank's own rows follow all of them
        owner = torch.bucketize(pos, plan.cut[1:].contiguous(), right=True)
        arriving = [(self.rank + k) % w for k in range(1, w) if plan.recv_counts[(self.rank + k) % w] > 0]
        groups = max(1, min(self.owner_groups, len(arriving))) if arriving else 0
        bundles = [()] + [tuple(arriving[g * len(arriving) // groups:(g + 1) * len(arriving) // groups])
                          for g in range(groups)]
        out = []
        for owners in bundles:
            pick = owner == w if not owners else torch.isin(owner, torch.tensor(owners, device=dev))
            count = int(pick.sum().item())
            tp = None
            if count:
                tp = self.capi.TilePlan.from_ids(rows[pick].to(torch.int32), pos[pick].to(torch.int32), count, n_loc,
                                                 num_sources=plan.num_rows)
            if owners and tp is None:
                continue
            out.append((owners, tp))
        cache[(kind, i)] = out
        return out

    def _segments_spmm(self, kind, i, buf, out, wait: bool):
        """The aggregation of one buffer, bundle by bundle: the rank's own sources are stored, the others
        added; with ``wait`` the stream first waits for the rows of a bundle's owners (streamed exchange)."""
        fab = self.fabric
        for owners, tp in self._segment_plans(kind, i):
            if not owners:
                if tp is None:
                    out.zero_()
                else:
                    self.capi.spmm_tiles(buf, tp, self.deg_row, out=out)
                continue
            if wait:
                fab.capi.wait_landed(fab.landed, owners, fab.epoch, fab.status, fab.max_polls)
            self.capi.spmm_tiles_add(buf, tp, self.deg_row, out)

    def _streamed_op(self, kind, i, local, out_local, plan, bufs):
        """Exchange and aggregation overlapped owner by owner (see :meth:`DealtHalo.start_streamed`), chunk
        after chunk.  Backward rows are multiplied by their source-side factor while they are placed."""
        if kind == "bwd":
            self.path[i].setdefault("prescaled", {})[bufs[0][1].size(1)] = True
        dc = out_local.size(1) // len(bufs)
        for c, (peers, buf) in enumerate(bufs):
            rows = None if local is None else local[:, c * dc:(c + 1) * dc]
            plan.start_streamed(rows, buf, peers, self.deg_row if kind == "bwd" else None)
            self._segments_spmm(kind, i, buf, out_local[:, c * dc:(c + 1) * dc], wait=True)
            plan.end_streamed()
        return out_local

    def _dealt_op(self, kind, i, local, out_local):
        """Chunked exchange + aggregation: chunk ``c`` is aggregated (straight into
        its column block of ``out_local``) while chunk ``c + 1`` travels.  A backward
        layer's rows are multiplied by their source-side factor while they are copied
        into the exchange buffer (every rank scales the rows it owns), so that the
        aggregation runs the tile kernel on pre-scaled rows; that needs the caller's
        rows (``local``) and 16-byte aligned buffer rows, else the group kernel
        applies the factor per edge."""
        plan = self.fwd_plan if kind == "fwd" else self.path[i]["plan"]
        scale = None
        if self.streamed and (kind == "fwd" or local is not None):
            bufs = plan.buffers(out_local.size(1), self.chunks)
            if all(self._tiles_can_read(b) for _, b in bufs):
                return self._streamed_op(kind, i, local, out_local, plan, bufs)
        if kind == "bwd":
            d = out_local.size(1)
            bufs = plan.buffers(d, self.chunks)
            aligned = all(self._tiles_can_read(b) for _, b in bufs)
            p = self.path[i]
            want = local is not None and aligned
            # remembered per buffer width: the kernels-only timing path re-runs the aggregation on the buffers
            # as the last exchange left them
            p.setdefault("prescaled", {})[bufs[0][1].size(1)] = want
            scale = self.deg_row if want else None
        pending = plan.start(local, self.chunks, out_local.size(1), scale=scale)
        dc = out_local.size(1) // len(pending)
        for c, (work, buf) in enumerate(pending):
            if work is not None:
                work.wait()
            self._halo_spmm(kind, i, buf, out_local[:, c * dc:(c + 1) * dc])
        return out_local

    def graphed(self, fn, warmup: int = 2):
        """Captures the launches of ``fn()`` (aggregations of this object on fixed tensors) into a CUDA
        graph and returns a callable that replays them: one submission per step instead of a dozen, which
        keeps the ranks in step with one another between the flag barriers.  Only this library's kernels
        and peer stores are captured; with a transport that calls NCCL, or on the CPU, ``fn`` itself is
        returned.  ``fn`` must be the steady state: it runs ``warmup`` times first (plans are built and the
        exchange's barrier bookkeeping settles), every rank must capture and replay the same sequence,
        and between replays no other aggregation of this object may run."""
        dev = torch.device(self.dev)
        if dev.type != "cuda" or (self.world > 1 and self.fabric is None):
            return fn
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):
                fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        _sync(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            fn()
        _sync(dev)
        self.__dict__.setdefault("_graphs", []).append(graph)
        return graph.replay

    def halo_inputs(self, kind, i, d):
        """Where the producer of an aggregation's input puts this rank's rows (see
        :meth:`DealtHalo.own_rows`); pass ``None`` as the input afterwards."""
        plan = self.fwd_plan if kind == "fwd" else self.path[i]["plan"]
        return plan.own_rows(d, self.chunks)

    def check(self):
        """Raises if a bounded wait of the peer-store transport ran out.  After such a
        time-out later barriers no longer wait and the exchange buffers may be half
        filled, so results must not be trusted: call this at a point where a host
        synchronisation is affordable (once per epoch, or before results leave the
        rank).  A no-op for the NCCL transports, whose errors surface as exceptions."""
        if self.fabric is not None:
            self.fabric.check()

    def halo_local(self, kind, i, out_local):
        """Only the aggregation kernels of one operation, on the buffers the last exchange filled."""
        plan = self.fwd_plan if kind == "fwd" else self.path[i]["plan"]
        bufs = plan.buffers(out_local.size(1), self.chunks)
        dc = out_local.size(1) // len(bufs)
        streamed = self.streamed and all(self._tiles_can_read(b) for _, b in bufs) and \
            (kind == "fwd" or self.path[i].get("prescaled", {}).get(bufs[0][1].size(1)))
        for c, (_, buf) in enumerate(bufs):
            if streamed:
                self._segments_spmm(kind, i, buf, out_local[:, c * dc:(c + 1) * dc], wait=False)
            else:
                self._halo_spmm(kind, i, buf, out_local[:, c * dc:(c + 1) * dc])

    def forward_halo(self, local, out_local):
        """Exchange of the referenced (pre-scaled) source rows, then the local forward aggregation."""
        if isinstance(self.fwd_plan, DealtHalo):
            return self._dealt_op("fwd", 0, local, out_local)
        buf = self.fwd_plan.exchange(local)
        return self._halo_spmm("fwd", 0, buf, out_local)

    def backward_halo(self, i, d_out_local, out_local):
        p = self.path[i]
        if isinstance(p["plan"], DealtHalo):
            return self._dealt_op("bwd", i, d_out_local, out_local)
        buf = p["plan"].exchange(d_out_local)
        return self.capi.spmm_backward_compacted(buf, p["id"], p["pp"], p["edges_c"], p["deg_c"], p["parts"],
                                                 self.back_size, out=out_local, deg_row=self.deg_row,
                                                 num_rows=self.shard.num_rows)
