"""Aggregation on two real GPUs (NCCL) against the float64 oracle of the whole
graph, in every partition/exchange mode and transport.  Skipped on a machine
with fewer than two GPUs."""
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, results):
    import os
    os.environ["NCCL_NVLS_ENABLE"] = "0"          # plain peer transport is all this test needs
    from eppgcn_b200 import dist as D
    from eppgcn_b200 import graphs
    from oracle import epp_oracle as O
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=dev)
    try:
        ds = graphs.load_workload("pubmed", 0)
        g, n = ds.graph, ds.num_nodes
        deg = ds.degrees.numpy().copy()
        train = ds.train_mask.numpy().copy()
        parts = mode.split(":")                                        # "balanced_halo:2:nccl[:graph|overlap]"
        mode, chunks, transport = parts[0], (parts[1:2] or ["1"])[0], (parts[2:3] or ["push"])[0]
        extra = (parts[3:4] or [""])[0]
        hp = D.DistHotPath(ds, dev, rank, world, back_size=8, exchange=mode, chunks=int(chunks), transport=transport,
                           overlap=extra == "overlap", streamed="stream" in extra)
        graph = "graph" in extra
        sh = hp.shard
        rng = np.random.Generator(np.random.PCG64(11))
        mats = [rng.standard_normal((n, d)).astype(np.float32) for d in (16, 22)]
        # this rank's rows of a whole-graph matrix, in the partition's own numbering
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
            return torch.from_numpy(out).to(dev)

        path, _ = O.prepare_execution_path(g.indptr, g.indices, train, 2, hp.part_size, [8, 8])
        ok = True
        for m in mats:
            d = m.shape[1]
            scaled = local_rows(m * deg[:, None])                       # rows as the update step leaves them
            out = torch.empty(sh.num_rows, d, device=dev)
            dist.barrier()          # the oracle work between the steps differs per rank: line the ranks up again
            if mode in ("halo", "balanced_halo"):
                hp.forward_halo(scaled, out)
            else:
                full = torch.empty(hp.n, d, device=dev)
                hp.gather(full, scaled)
                hp.forward(full, out)
            want = O.spmm_forward(g.indptr, g.indices, deg, m)
            err = np.abs(out.cpu().numpy()[have] - want[mine[have]]) - (2e-6 + 2e-5 * np.abs(want[mine[have]]))
            ok &= bool(err.max() <= 0)
            for i, conv in enumerate(path):
                d_in = torch.empty(sh.num_rows, d, device=dev)
                dist.barrier()
                if "plan" in hp.path[i]:
                    hp.backward_halo(i, local_rows(m), d_in)
                else:
                    full = torch.empty(hp.n, d, device=dev)
                    hp.gather(full, local_rows(m))
                    hp.backward(i, full, d_in)
                wb = O.ours_backward_aggregate(conv["id"], conv["partPointer"], conv["edgeList"], deg, m,
                                               conv["numParts"])
                err = np.abs(d_in.cpu().numpy()[have] - wb[mine[have]]) - (2e-6 + 2e-5 * np.abs(wb[mine[have]]))
                ok &= bool(err.max() <= 0)
        if graph:
            # one forward and one compacted backward aggregation captured into a CUDA graph and replayed on new
            # inputs: the barriers number themselves on the device, so every replay lines the ranks up again
            d = 16
            x_in = torch.zeros(sh.num_rows, d, device=dev)
            b_in = torch.zeros(sh.num_rows, d, device=dev)
            f_out = torch.empty(sh.num_rows, d, device=dev)
            b_out = torch.empty(sh.num_rows, d, device=dev)

            def step():
                hp.forward_halo(x_in, f_out)
                hp.backward_halo(0, b_in, b_out)

            run = hp.graphed(step)
            ok &= run is not step
            for _ in range(3):
                m = rng.standard_normal((n, d)).astype(np.float32)
                x_in.copy_(local_rows(m * deg[:, None]))
                b_in.copy_(local_rows(m))
                run()
                want = O.spmm_forward(g.indptr, g.indices, deg, m)
                err = np.abs(f_out.cpu().numpy()[have] - want[mine[have]]) - (2e-6 + 2e-5 * np.abs(want[mine[have]]))
                ok &= bool(err.max() <= 0)
                conv = path[0]
                wb = O.ours_backward_aggregate(conv["id"], conv["partPointer"], conv["edgeList"], deg, m,
                                               conv["numParts"])
                err = np.abs(b_out.cpu().numpy()[have] - wb[mine[have]]) - (2e-6 + 2e-5 * np.abs(wb[mine[have]]))
                ok &= bool(err.max() <= 0)
        # the sharded path sizes add up to the single-process ones
        sizes = torch.tensor([p["valid"] for p in hp.path] + [p["parts"] for p in hp.path], device=dev)
        dist.all_reduce(sizes)
        ok &= sizes[:2].tolist() == [c["valid_len"] for c in path]
        if hp.fabric is not None:
            hp.fabric.check()                         # no bounded wait ran out
            ok &= hp.fabric.count > 0
            ok &= (int(hp.fabric.epoch.item()) > 0) == hp.streamed
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("mode", ["balanced", "allgather", "halo", "balanced_halo", "balanced_halo:2", "balanced_halo:2:nccl",
                                  "balanced_halo:1:push:graph", "balanced_halo:2:push:overlap", "balanced_halo:1:push:stream",
                                  "balanced_halo:2:push:stream+graph"])
def test_two_gpus_match_the_whole_graph_oracle(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mgr = mp.get_context("spawn").Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), mode, results), nprocs=2, join=True)
    assert dict(results) == {0: True, 1: True}
