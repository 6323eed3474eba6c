"""The whole multi-rank orchestration on two gloo ranks without a GPU.

``DistHotPath`` is run on CPU tensors with the device entry points replaced by
a test double built from the oracle (numpy).  Everything around the kernels is
the real code: relabelling, shards, sharded path marking with the mask
reduction, compaction and splitting per shard, the exchange plans of every mode
(re-indexed edge lists, degree vectors in buffer order, column chunks) and the
collectives.  Each rank's results are checked against the float64 oracle of the
whole graph.  The kernels themselves are checked on GPUs elsewhere."""
import contextlib

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.test_dist import free_port


def _install_oracle_double():
    """Replaces the device entry points ``DistHotPath`` calls with numpy
    restatements that take and return CPU tensors."""
    from eppgcn_b200 import capi
    from oracle import epp_oracle as O

    def mask_forward(ids, part_ptr, edge_list, src_mask, ngh_mask, back_edge_mask, node_degs, num_layers, layer,
                     blockx=4, blocky=16, row_offset=0):
        n = src_mask.numel()
        degs = np.zeros(n, dtype=np.int32)
        degs[row_offset:row_offset + node_degs.numel()] = node_degs.numpy()
        ngh = ngh_mask.numpy() if ngh_mask is not None else np.zeros(0, dtype=bool)
        marks = back_edge_mask.numpy()
        fresh = marks == -1
        O.mask_forward(ids.numpy().astype(np.int64) + row_offset, part_ptr.numpy(), edge_list.numpy(),
                       src_mask.numpy(), ngh, marks, degs, num_layers, layer)
        marks[fresh & (marks != -1)] -= row_offset            # the device kernel records the shard's own row numbers
        node_degs.copy_(torch.from_numpy(degs[row_offset:row_offset + node_degs.numel()]))

    def compact_mask(edge_mask, col_idx, mode=0):
        ids, cols, valid = O.compact_back_edge(edge_mask.numpy(), col_idx.numpy())
        return (torch.from_numpy(np.asarray(ids, dtype=np.int32)), torch.from_numpy(np.asarray(cols, dtype=np.int32)),
                int(valid))

    def split_parts(node_deg, num_edges, part_size, mode=0, out_len=None):
        pp, parts = O.split_back_part(node_deg.numpy(), num_edges, part_size, out_len=num_edges + 1)
        return torch.from_numpy(np.asarray(pp, dtype=np.int32)), int(parts)

    def spmm_forward(feat, row_ptr, col_idx, degrees, part_ptr, part2node, part_size=0, dim_worker=32,
                     warp_per_block=8, out=None, deg_row=None, prescaled=False):
        ptr, col = row_ptr.numpy().astype(np.int64), col_idx.numpy().astype(np.int64)
        rows = np.repeat(np.arange(len(ptr) - 1), np.diff(ptr))
        src = feat.numpy().astype(np.float64)[col]
        if not prescaled:
            src = src * degrees.numpy().astype(np.float64)[col][:, None]
        acc = np.zeros((len(ptr) - 1, feat.size(1)))
        np.add.at(acc, rows, src)
        acc *= (degrees if deg_row is None else deg_row).numpy().astype(np.float64)[:len(ptr) - 1, None]
        out.copy_(torch.from_numpy(acc.astype(np.float32)))
        return out

    def spmm_backward_compacted(d_out, ids, part_ptr, edge_list, degrees, num_parts, part_size=0, blockx=4,
                                blocky=16, out=None, deg_row=None, num_rows=None):
        valid = int(part_ptr[num_parts]) if num_parts > 0 else 0
        r, c = ids.numpy()[:valid].astype(np.int64), edge_list.numpy()[:valid].astype(np.int64)
        dr = (degrees if deg_row is None else deg_row).numpy().astype(np.float64)
        w = dr[r] * degrees.numpy().astype(np.float64)[c]
        acc = np.zeros((out.size(0), d_out.size(1)))
        np.add.at(acc, r, d_out.numpy().astype(np.float64)[c] * w[:, None])
        out.copy_(torch.from_numpy(acc.astype(np.float32)))
        return out

    class TilePlan:
        """Double of the tiled kernel's plan: just remembers the edge list as (row, source) pairs."""

        def __init__(self, rows, cols, num_rows):
            self.rows, self.cols, self.num_rows = rows, cols, num_rows

        @classmethod
        def from_csr(cls, row_ptr, col_idx, num_sources=None):
            assert num_sources is None or col_idx.numel() == 0 or int(col_idx.max()) < num_sources
            ptr = row_ptr.numpy().astype(np.int64)
            return cls(np.repeat(np.arange(len(ptr) - 1), np.diff(ptr)), col_idx.numpy().astype(np.int64), len(ptr) - 1)

        @classmethod
        def from_ids(cls, ids, col_idx, num_edges, num_rows, num_sources=None):
            assert num_sources is None or num_edges == 0 or int(col_idx[:num_edges].max()) < num_sources
            return cls(ids.numpy()[:num_edges].astype(np.int64), col_idx.numpy()[:num_edges].astype(np.int64), num_rows)

    def spmm_tiles(src, plan, row_scale=None, out=None):
        acc = np.zeros((plan.num_rows, src.size(1)))
        np.add.at(acc, plan.rows, src.numpy().astype(np.float64)[plan.cols])
        if row_scale is not None:
            acc *= row_scale.numpy().astype(np.float64)[:plan.num_rows, None]
        out.copy_(torch.from_numpy(acc.astype(np.float32)))
        return out

    def spmm_tiles_add(src, plan, row_scale, out):
        acc = np.zeros((plan.num_rows, src.size(1)))
        np.add.at(acc, plan.rows, src.numpy().astype(np.float64)[plan.cols])
        if row_scale is not None:
            acc *= row_scale.numpy().astype(np.float64)[:plan.num_rows, None]
        out.add_(torch.from_numpy(acc.astype(np.float32)))
        return out

    def pack_scaled_rows(x, scale, plan=None, out=None, pad_to=8):
        assert plan is None
        out.copy_(x * scale[:, None])
        return out

    for name, fn in dict(mask_forward=mask_forward, compact_mask=compact_mask, split_parts=split_parts,
                         spmm_forward=spmm_forward, spmm_backward_compacted=spmm_backward_compacted,
                         spmm_tiles=spmm_tiles, spmm_tiles_add=spmm_tiles_add, TilePlan=TilePlan,
                         pack_scaled_rows=pack_scaled_rows).items():
        setattr(capi, name, fn)


class SharedFileFabric:
    """Stand-in for ``PeerFabric`` on CPU ranks of one machine: a buffer is a
    file in shared memory that every rank maps, "peer addresses" are the mapped
    tensors themselves, the push is an indexed copy into them and the barrier is
    the process group's.  For the streamed exchange the "landed" words are one more shared file, the
    signalling push writes them after its rows, and the wait polls them.  Same members as the real
    one, so the plans run unchanged."""

    tag = "0"

    def __init__(self, dev, rank, world, group=None):
        import types
        self.rank, self.world, self.group = rank, world, group
        self.count, self.files, self.keep = 0, [], []
        self.capi = types.SimpleNamespace(push_rows=self.push_rows, push_rows_signal=self.push_rows_signal,
                                          bump_counter=self.bump_counter, wait_landed=self.wait_landed)
        self._landed = None                            # allocated at first use: the constructor has no collective
        self.epoch = torch.zeros(1, dtype=torch.int32)
        self.done = torch.zeros(16, dtype=torch.int32)
        self.status = torch.zeros(1, dtype=torch.int32)
        self.max_polls = 20_000
        self.signals = 0

    @staticmethod
    def available(dev, group=None):
        return True

    @property
    def landed(self):
        if self._landed is None:
            self._landed = self.alloc((64,), torch.int32)
        return self._landed[0]

    @property
    def landed_ptrs(self):
        self.landed
        return self._landed[1]

    def alloc(self, shape, dtype=torch.float32):
        import os
        np_dtype = {torch.float32: np.float32, torch.int32: np.int32}[dtype]
        index = len(self.files)
        names = [f"/dev/shm/eppgcn_test_{self.tag}_{index}_{r}" for r in range(self.world)]
        own = np.lib.format.open_memmap(names[self.rank], mode="w+", dtype=np_dtype, shape=tuple(shape))
        own[...] = 0
        own.flush()
        dist.barrier(self.group)
        maps = [own if r == self.rank else np.load(names[r], mmap_mode="r+") for r in range(self.world)]
        dist.barrier(self.group)
        os.unlink(names[self.rank])                   # the mappings keep the memory alive; nothing is left behind
        self.files.append(names)
        self.keep.append(maps)
        tensors = [torch.from_numpy(m) for m in maps]
        return tensors[self.rank], tensors

    def push_rows(self, rows, send_idx, send_ptr, peers, first_row, dim, start_row=0):
        assert rows.size(1) == dim and dim % 4 == 0 and 0 <= start_row < max(send_ptr[-1], 1)
        for r, peer in enumerate(peers):
            lo, hi = send_ptr[r], send_ptr[r + 1]
            if hi > lo:
                peer[first_row[r]:first_row[r] + hi - lo, :dim] = rows[send_idx[lo:hi].long()]

    def push_rows_signal(self, rows, send_idx, send_ptr, peers, first_row, dim, rank, landed, epoch, done):
        assert rank == self.rank and send_ptr[rank] == send_ptr[rank + 1]
        for k in range(1, self.world):                 # served leftwards from the rank, like the kernel
            r = (rank - k) % self.world
            lo, hi = send_ptr[r], send_ptr[r + 1]
            if hi > lo:
                peers[r][first_row[r]:first_row[r] + hi - lo, :dim] = rows[send_idx[lo:hi].long()]
                landed[r][rank] = int(epoch[0])
                self.signals += 1

    @staticmethod
    def bump_counter(counter):
        counter += 1

    def wait_landed(self, landed, owners, epoch, status, max_polls):
        import time
        for r in owners:
            polls = 0
            while int(landed[r]) - int(epoch[0]) < 0:
                polls += 1
                assert polls < max_polls, "the rows of another rank never arrived"
                time.sleep(0.001)

    @contextlib.contextmanager
    def side_stream(self):
        yield

    def join_side_stream(self):
        pass

    def barrier(self):
        self.count += 1
        dist.barrier(self.group)

    def check(self):
        pass


def _worker(rank, world, port, mode, results):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        _install_oracle_double()
        from eppgcn_b200 import dist as D
        from eppgcn_b200 import graphs
        from oracle import epp_oracle as O
        parts = mode.split(":")
        mode, chunks = parts[0], int((parts[1:2] or ["1"])[0])
        if parts[2:3] == ["push"]:                    # the peer-store transport, on files in shared memory
            SharedFileFabric.tag = str(port)
            D.PeerFabric = SharedFileFabric
        if parts[2:3] == ["broken"]:                  # peer buffers fail on one rank only: all ranks must fall back
            class Broken(SharedFileFabric):
                def __init__(self, dev, rank, world, group=None):
                    if rank == 1:
                        raise RuntimeError("no peer access")
                    super().__init__(dev, rank, world, group)
            D.PeerFabric = Broken
        ds = graphs.load_workload("cora", 0, layers=3)
        g, n = ds.graph, ds.num_nodes
        deg, train = ds.degrees.numpy().copy(), ds.train_mask.numpy().copy()
        streamed = parts[3:4] == ["streamed"]
        hp = D.DistHotPath(ds, torch.device("cpu"), rank, world, back_size=4, exchange=mode, chunks=chunks,
                           streamed=streamed, owner_groups=int((parts[4:5] or ["0"])[0]))
        sh = hp.shard
        if hp.new_of_old is not None:
            old_of_new = np.full(hp.n, -1, dtype=np.int64)
            old_of_new[hp.new_of_old] = np.arange(n)
            mine = old_of_new[sh.v0:sh.v1]
        else:
            mine = np.arange(sh.v0, sh.v1)
        have = mine >= 0

        def local_rows(m):
            out = np.zeros((sh.num_rows, m.shape[1]), dtype=np.float32)
            out[have] = m[mine[have]]
            return torch.from_numpy(out)

        def close(got, want):
            got, want = got.numpy()[have], want[mine[have]]
            return bool((np.abs(got - want) - (2e-6 + 2e-5 * np.abs(want))).max() <= 0)

        path, _ = O.prepare_execution_path(g.indptr, g.indices, train, 3, hp.part_size, [4, 4, 4])
        sizes = torch.tensor([p["valid"] for p in hp.path] + [p["parts"] for p in hp.path])
        dist.all_reduce(sizes)
        ok = sizes[:3].tolist() == [c["valid_len"] for c in path]
        rng = np.random.Generator(np.random.PCG64(11))
        for d in (16, 22):
            m = rng.standard_normal((n, d)).astype(np.float32)
            out = torch.empty(sh.num_rows, d)
            if mode in ("halo", "balanced_halo"):
                hp.forward_halo(local_rows(m * deg[:, None]), out)
            else:
                full = torch.empty(hp.n, d)
                hp.gather(full, local_rows(m * deg[:, None]))
                hp.forward(full, out)
            ok &= close(out, O.spmm_forward(g.indptr, g.indices, deg, m))
            for i, conv in enumerate(path):
                d_in = torch.empty(sh.num_rows, d)
                if "plan" in hp.path[i]:
                    hp.backward_halo(i, local_rows(m), d_in)
                else:
                    full = torch.empty(hp.n, d)
                    hp.gather(full, local_rows(m))
                    hp.backward(i, full, d_in)
                ok &= close(d_in, O.ours_backward_aggregate(conv["id"], conv["partPointer"], conv["edgeList"], deg, m,
                                                            conv["numParts"]))
        step = lambda: None                          # noqa: E731
        ok &= hp.graphed(step) is step                # nothing to capture without a CUDA device
        if parts[2:3] == ["push"]:
            ok &= isinstance(hp.fabric, SharedFileFabric) and hp.fabric.count > 0
            ok &= hp.fabric.signals > 0 if streamed else hp.fabric.signals == 0
        if parts[2:3] == ["broken"]:
            ok &= hp.fabric is None
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("mode", ["balanced", "allgather", "halo", "balanced_halo", "balanced_halo:2",
                                  "balanced_halo:1:push", "balanced_halo:2:push", "balanced_halo:1:push:streamed",
                                  "balanced_halo:2:push:streamed",
                                  "balanced_halo:1:broken"])
def test_two_gloo_ranks_match_the_whole_graph_oracle(mode):
    world = 2
    mgr = mp.get_context("spawn").Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, free_port(), mode, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


@pytest.mark.timeout(600)
def test_three_ranks_and_a_vertex_count_that_does_not_divide(tmp_path):
    """Cora has 2,708 vertices: three ranks need padding rows in the last block."""
    world = 3
    mgr = mp.get_context("spawn").Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, free_port(), "balanced_halo:2:push", results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True, 2: True}


@pytest.mark.timeout(600)
def test_four_ranks_with_the_owners_bundled_into_two_groups():
    """The streamed exchange with more owners than groups: three arriving owners in two bundles."""
    world = 4
    mgr = mp.get_context("spawn").Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, free_port(), "balanced_halo:1:push:streamed:2", results), nprocs=world, join=True)
    assert dict(results) == {r: True for r in range(world)}
