"""Host-side failure cases of the row-partitioned path on gloo ranks (CPU): ranks that disagree on
the partition raise on every rank with the field named, and a rank that leaves between steps
surfaces as an exception on the others instead of a hang.  No GPU is involved; nothing is made to
fault or hang."""
import datetime
import time

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from eppgcn_b200 import dist as D
from tests.test_dist import free_port


def _disagree(rank, world, port, results):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        D.check_agreement({"the vertex count": 2708, "the layer count": 2})          # all equal: passes
        try:
            D.check_agreement({"the vertex count": 2708, "the edge count": 13264 + (rank == 1), "the layer count": 2})
            results[rank] = "no error"
        except RuntimeError as exc:
            results[rank] = str(exc)
    finally:
        dist.destroy_process_group()


def test_ranks_that_disagree_on_the_partition_raise_everywhere():
    world = 3
    results = mp.Manager().dict()
    mp.spawn(_disagree, args=(world, free_port(), results), nprocs=world, join=True)
    for r in range(world):
        assert "disagree on the edge count" in results[r], results[r]
        assert "rank 1: 13265" in results[r] and "rank 0: 13264" in results[r]


def _hot_path_disagree(rank, world, port, results):
    """The real constructor: rank 1 is given another train ratio, i.e. another execution path."""
    from eppgcn_b200 import graphs
    from tests.test_dist_end_to_end import _install_oracle_double
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        _install_oracle_double()
        ds = graphs.load_workload("cora", 0, train_ratio=0.1 if rank == 0 else 0.3)
        try:
            D.DistHotPath(ds, torch.device("cpu"), rank, world, 8, exchange="balanced")
            results[rank] = "no error"
        except RuntimeError as exc:
            results[rank] = str(exc)
    finally:
        dist.destroy_process_group()


def test_the_hot_path_refuses_ranks_with_different_train_masks():
    results = mp.Manager().dict()
    mp.spawn(_hot_path_disagree, args=(2, free_port(), results), nprocs=2, join=True)
    assert all("disagree on the train-mask size" in results[r] for r in range(2)), dict(results)


def _leaver(rank, world, port, results):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8))
    n = 64
    bounds = np.array([0, n // 2, n], dtype=np.int64)
    rows = torch.full((n // 2, 8), float(rank))
    full = torch.zeros(n, 8)
    D.all_gather_rows(full, rows, bounds)                     # step 1: everybody is there
    ok = bool((full[: n // 2] == 0).all() and (full[n // 2:] == 1).all())
    if rank == 1:                                              # leaves between steps, nothing in flight
        results[rank] = "left" if ok else "bad first step"
        dist.destroy_process_group()
        return
    t0 = time.time()
    try:
        D.all_gather_rows(full, rows, bounds)                 # step 2: the peer is gone
        results[rank] = "no error"
    except Exception as exc:                                   # noqa: BLE001 - any exception type will do, a hang will not
        results[rank] = f"raised after {time.time() - t0:.1f}s: {type(exc).__name__}"
    try:
        dist.destroy_process_group()
    except Exception:                                          # noqa: BLE001
        pass


def test_a_rank_that_leaves_between_steps_surfaces_as_an_exception():
    results = mp.Manager().dict()
    mp.spawn(_leaver, args=(2, free_port(), results), nprocs=2, join=True)
    assert results[1] == "left"
    assert results[0].startswith("raised after"), results[0]
    assert float(results[0].split()[2][:-2]) < 30.0
