"""Row-partition logic on two gloo ranks (CPU): ranges, shards, the row
exchange, and the sharded execution-path preparation against the
single-process oracle."""
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from eppgcn_b200 import dist as D
from eppgcn_b200 import graphs
from oracle import epp_oracle as O


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_edge_balanced_ranges():
    g = graphs.make_graph("pubmed", 0, cache=False)
    for world in (1, 2, 3, 8):
        b = D.edge_balanced_ranges(g.indptr, world)
        assert b[0] == 0 and b[-1] == g.num_nodes and np.all(np.diff(b) >= 0) and len(b) == world + 1
        edges = np.diff(g.indptr[b].astype(np.int64))
        assert edges.sum() == g.num_edges
        assert edges.max() - g.num_edges / world <= np.diff(g.indptr).max()     # off by at most one row
    # a hub bigger than its share still leaves valid (possibly empty) ranges
    hub = np.array([0, 100, 101, 102, 103], dtype=np.int32)
    b = D.edge_balanced_ranges(hub, 4)
    assert b[0] == 0 and b[-1] == 4 and np.all(np.diff(b) >= 0)


def test_shards_tile_the_graph():
    g = graphs.make_graph("cora", 0, cache=False)
    b = D.edge_balanced_ranges(g.indptr, 3)
    shards = [D.make_shard(g.indptr, g.indices, b, r) for r in range(3)]
    assert sum(s.num_rows for s in shards) == g.num_nodes
    assert np.array_equal(np.concatenate([s.indices for s in shards]), g.indices)
    for s in shards:
        assert s.indptr[0] == 0 and s.indptr[-1] == s.num_edges
        assert np.array_equal(np.diff(s.indptr), np.diff(g.indptr[s.v0:s.v1 + 1]))


def _worker(rank, world, port, results):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        g = graphs.make_graph("cora", 0, cache=False)
        n, e = g.num_nodes, g.num_edges
        bounds = D.edge_balanced_ranges(g.indptr, world)
        sh = D.make_shard(g.indptr, g.indices, bounds, rank)
        # --- row exchange into a padded buffer -----------------------------------------
        want = torch.arange(n * 22, dtype=torch.float32).reshape(n, 22)
        full = torch.full((n, 24), -1.0)[:, :22]
        D.all_gather_rows(full, want[sh.v0:sh.v1].clone(), bounds)
        ok_gather = bool(torch.equal(full, want))
        # --- sharded preparation: local marking + OR-reduced neighbour masks -----------
        layers, ps, bs = 3, 4, 8
        train = np.random.Generator(np.random.PCG64(7)).random(n) < 0.1
        pp, p2n = O.build_part(ps, sh.indptr)
        ngh = [torch.zeros(n, dtype=torch.bool) for _ in range(layers - 1)]
        ems = [np.full(sh.num_edges, -1, dtype=np.int32) for _ in range(layers)]
        nds = [np.zeros(n, dtype=np.int32) for _ in range(layers)]          # indexed by global row here
        for i in range(layers):
            src = train if i == 0 else ngh[i - 1].numpy()
            dst = ngh[i].numpy() if i < layers - 1 else np.zeros(0, dtype=bool)
            O.mask_forward(p2n.astype(np.int64) + sh.v0, pp, sh.indices, src, dst, ems[layers - 1 - i],
                           nds[layers - 1 - i], layers, i + 1)
            if i < layers - 1:
                D.or_reduce_mask(ngh[i])
        ref, ref_ngh = O.prepare_execution_path(g.indptr, g.indices, train, layers, ps, [bs] * layers)
        e0, e1 = int(g.indptr[sh.v0]), int(g.indptr[sh.v1])
        ok_prep = all(np.array_equal(ngh[i].numpy(), ref_ngh[i]) for i in range(layers - 1))
        for i in range(layers):
            ok_prep &= np.array_equal(ems[i], ref[i]["edge_mask"][e0:e1])
            ok_prep &= np.array_equal(nds[i][sh.v0:sh.v1], ref[i]["node_degs"][sh.v0:sh.v1])
            # the shard's compacted list is the matching slice of the global one
            ids, cols, valid = O.compact_back_edge(ems[i], sh.indices)
            before = int((ref[i]["edge_mask"][:e0] != -1).sum())
            ok_prep &= np.array_equal(ids[:valid], ref[i]["id"][before:before + valid])
            ok_prep &= np.array_equal(cols[:valid], ref[i]["edgeList"][before:before + valid])
        # --- halo exchange: only referenced rows travel, edges are re-indexed -----------------
        plan = D.HaloPlan(torch.from_numpy(sh.indices), bounds, rank, world)
        local_rows = torch.full((sh.num_rows, 24), -1.0)[:, :22]
        local_rows.copy_(want[sh.v0:sh.v1])
        buf = plan.exchange(local_rows)
        ok_halo = bool(torch.equal(buf[plan.remap.long()], want[torch.from_numpy(sh.indices).long()]))
        ok_halo &= plan.num_rows == len(np.unique(sh.indices)) and buf.stride(0) == 24
        ok_halo &= bool(torch.equal(plan.needed, torch.from_numpy(np.unique(sh.indices)).long()))
        # --- masked-row exchange over equal blocks (backward layers of the balanced mode) -----
        n_eq = (n // world) * world
        mask = torch.from_numpy(np.random.Generator(np.random.PCG64(3)).random(n_eq) < 0.2)
        mg = D.MaskedGather(mask, n_eq // world, rank, world)
        blk = n_eq // world
        buf = mg.exchange(want[rank * blk:(rank + 1) * blk].clone())
        sel = torch.nonzero(mask).view(-1)
        ok_halo &= bool(torch.equal(buf[mg.pos[sel].long()], want[sel]))
        ok_halo &= mg.num_rows == world * mg.cap and mg.cap == int(mask.view(world, blk).sum(1).max())
        ok_halo &= bool(torch.equal(mg.compact(torch.arange(n_eq, dtype=torch.float32))[mg.pos[sel].long()], sel.float()))
        # --- dealt halo: remote referenced rows by all-to-all in column chunks, own rows in place ----
        new_of_old, n_eqr = D.balanced_relabel(g.indptr, world)
        rsh = D.make_relabelled_shard(g.indptr, g.indices, new_of_old, n_eqr, rank, world)
        rcols = torch.from_numpy(rsh.indices)
        dh = D.DealtHalo(rcols, n_eqr, rank, world)
        whole = torch.arange(n_eqr * world * 24, dtype=torch.float32).reshape(n_eqr * world, 24)
        mine = torch.zeros(n_eqr, 26)[:, :24]
        mine.copy_(whole[rank * n_eqr:(rank + 1) * n_eqr])
        remote = np.unique(rsh.indices[(rsh.indices // n_eqr) != rank])
        ok_halo &= dh.num_remote == len(remote) and dh.recv_counts[rank] == 0
        for chunks in (1, 2, 5):                              # 5 does not split 24 columns: falls back to one chunk
            pending = dh.start(mine, chunks)
            ok_halo &= len(pending) == (chunks if chunks < 5 else 1)
            parts = []
            for work, buf in pending:
                if work is not None:
                    work.wait()
                parts.append(buf)
            got = torch.cat(parts, 1)
            ok_halo &= bool(torch.equal(got, whole[dh.order]))
            ok_halo &= bool(torch.equal(got[dh.remap.long()], whole[rcols.long()]))
        # a rank whose edges reference nothing (empty path), and one that references only its own rows
        lonely = D.DealtHalo(torch.zeros(0, dtype=torch.int32) if rank == 0 else
                             torch.arange(rank * n_eqr, rank * n_eqr + 5, dtype=torch.int32), n_eqr, rank, world)
        ok_halo &= lonely.num_remote == 0 and lonely.num_rows == n_eqr and sum(lonely.send_counts) == 0
        (work, buf), = lonely.start(mine, 1)
        if work is not None:
            work.wait()
        ok_halo &= bool(torch.equal(buf, mine)) and (rank == 0 or lonely.remap.tolist() == list(range(5)))
        # --- d_weight partials add up -----------------------------------------------------
        part = torch.full((4, 3), float(rank + 1))
        dist.all_reduce(part)
        ok_sum = bool(torch.all(part == sum(range(1, world + 1))))
        results[rank] = (ok_gather, bool(ok_prep), ok_sum, bool(ok_halo))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_ranks_gloo():
    world = 2
    mgr = mp.get_context("spawn").Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: (True, True, True, True), 1: (True, True, True, True)}


def test_balanced_relabel_gives_equal_rows_and_edges():
    g = graphs.make_graph("pubmed", 0, cache=False)
    n = g.num_nodes
    for world in (1, 2, 3, 8):
        new_of_old, n_loc = D.balanced_relabel(g.indptr, world)
        assert n_loc == -(-n // world) and len(np.unique(new_of_old)) == n and new_of_old.max() < world * n_loc
        old_of_new = np.full(world * n_loc, -1)
        old_of_new[new_of_old] = np.arange(n)
        edges = []
        for r in range(world):
            sh = D.make_relabelled_shard(g.indptr, g.indices, new_of_old, n_loc, r, world)
            assert sh.num_rows == n_loc and sh.indptr[0] == 0 and sh.indptr[-1] == sh.num_edges
            edges.append(sh.num_edges)
            for lr in range(0, n_loc, max(1, n_loc // 50)):
                old = old_of_new[r * n_loc + lr]
                got = sh.indices[sh.indptr[lr]:sh.indptr[lr + 1]]
                want = new_of_old[g.indices[g.indptr[old]:g.indptr[old + 1]]] if old >= 0 else np.zeros(0)
                assert np.array_equal(got, want)
        assert sum(edges) == g.num_edges
        assert max(edges) - min(edges) <= np.diff(g.indptr).max()       # hubs are dealt out evenly
