"""The two exchange kernels on one GPU: the row push with local buffers
standing in for the peers' ones, and the flag barrier including its bounded
wait (a flag that nobody sets makes it run out; the context stays usable)."""
import numpy as np
import pytest
import torch

from eppgcn_b200 import capi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("start", [0, 700, 1999])
@pytest.mark.parametrize("dim,pad", [(4, 0), (16, 0), (32, 8), (64, 0)])
def test_push_rows_places_every_row(cuda, dim, pad, start):
    rng = np.random.Generator(np.random.PCG64(dim))
    n, world = 5000, 3
    rows = torch.randn(n, dim + pad, device=cuda)[:, :dim]
    counts = [700, 0, 1300]                                   # the middle "rank" gets nothing
    idx = torch.from_numpy(rng.integers(0, n, sum(counts)).astype(np.int32)).to(cuda)
    send_ptr = [0] + np.cumsum(counts).tolist()
    first = [11, 0, 5]
    bufs = [torch.full((c + first[r] + 3, dim), -1.0, device=cuda) for r, c in enumerate(counts)]
    capi.push_rows(rows, idx, send_ptr, [b.data_ptr() for b in bufs], first, dim, start_row=start)
    torch.cuda.synchronize()
    for r, c in enumerate(counts):
        got = bufs[r]
        want = rows[idx[send_ptr[r]:send_ptr[r + 1]].long()]
        assert torch.equal(got[first[r]:first[r] + c], want)
        assert bool((got[:first[r]] == -1).all()) and bool((got[first[r] + c:] == -1).all())


def test_push_rows_rejects_ragged_rows(cuda):
    rows = torch.randn(8, 6, device=cuda)
    idx = torch.zeros(1, dtype=torch.int32, device=cuda)
    with pytest.raises(capi.EppError) as e:
        capi.push_rows(rows, idx, [0, 1], [rows.data_ptr()], [0], 6)
    assert e.value.status == capi.EPP_ERR_BAD_ARG
    wide = torch.randn(8, 8, device=cuda)
    with pytest.raises(capi.EppError) as e:                     # the walk must start inside the send list
        capi.push_rows(wide, idx, [0, 1], [wide.data_ptr()], [0], 8, start_row=1)
    assert e.value.status == capi.EPP_ERR_BAD_ARG


def test_barrier_passes_alone_and_reports_a_missing_peer(cuda):
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    mine = torch.zeros(64, dtype=torch.int32, device=cuda)
    other = torch.zeros(64, dtype=torch.int32, device=cuda)
    # a group of one: the rank's own word is all it waits for
    for value in (1, 2, 3):
        capi.peer_barrier([mine.data_ptr()], 0, value, status)
    torch.cuda.synchronize()
    assert status.item() == capi.EPP_OK and mine[0].item() == 3
    # two ranks, the other one never arrives: its word stays 0, the wait runs out
    mine.zero_()
    capi.peer_barrier([mine.data_ptr(), other.data_ptr()], 0, 1, status, max_polls=2000)
    torch.cuda.synchronize()
    assert status.item() == capi.EPP_ERR_PEER_TIMEOUT
    assert other[0].item() == 1                   # the arrival was announced before the wait
    # the other rank "arrives": the same barrier now passes
    status.zero_()
    mine[1] = 1
    capi.peer_barrier([mine.data_ptr(), other.data_ptr()], 0, 1, status, max_polls=2000)
    torch.cuda.synchronize()
    assert status.item() == capi.EPP_OK


def test_counted_barrier_numbers_itself(cuda):
    """The barrier that takes its number from a device word: passes alone, counts its launches (so a
    captured launch can be replayed), and reports a peer that never arrives like the numbered one."""
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    counter = torch.zeros(1, dtype=torch.int32, device=cuda)
    mine = torch.zeros(64, dtype=torch.int32, device=cuda)
    other = torch.zeros(64, dtype=torch.int32, device=cuda)
    for _ in range(3):
        capi.peer_barrier_counted([mine.data_ptr()], 0, counter, status)
    torch.cuda.synchronize()
    assert status.item() == capi.EPP_OK and mine[0].item() == 3 and counter.item() == 3
    # replayed from a graph: every replay is the next barrier of the sequence
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=cuda)
    with torch.cuda.graph(graph, stream=side):
        capi.peer_barrier_counted([mine.data_ptr()], 0, counter, status)
    for _ in range(4):
        graph.replay()
    torch.cuda.synchronize()
    assert status.item() == capi.EPP_OK and mine[0].item() == 7 and counter.item() == 7
    # two ranks, the other one never arrives: the wait runs out, the arrival was announced
    capi.peer_barrier_counted([mine.data_ptr(), other.data_ptr()], 0, counter, status, max_polls=2000)
    torch.cuda.synchronize()
    assert status.item() == capi.EPP_ERR_PEER_TIMEOUT and other[0].item() == 8 and counter.item() == 8


@pytest.mark.parametrize("dim", [4, 16, 24, 64])
def test_signalling_push_places_every_row_and_tells_the_served_peers(cuda, dim):
    """Rank 1 of four pushes to local stand-ins of the peers' buffers: rows land as with the plain push,
    word 1 of every served peer's "landed" array carries the epoch, the peer without rows hears nothing,
    and the scratch counters are left zeroed (two exchanges in a row)."""
    rng = np.random.Generator(np.random.PCG64(dim))
    n, world, rank = 6000, 4, 1
    rows = torch.randn(n, dim, device=cuda)
    counts = [900, 0, 0, 1500]                                  # nothing for itself, nothing for rank 2
    idx = torch.from_numpy(rng.integers(0, n, sum(counts)).astype(np.int32)).to(cuda)
    send_ptr = [0] + np.cumsum(counts).tolist()
    first = [7, 0, 0, 3]
    bufs = [torch.full((c + first[r] + 2, dim), -1.0, device=cuda) for r, c in enumerate(counts)]
    landed = [torch.zeros(64, dtype=torch.int32, device=cuda) for _ in range(world)]
    epoch = torch.zeros(1, dtype=torch.int32, device=cuda)
    done = torch.zeros(16, dtype=torch.int32, device=cuda)
    for turn in (1, 2):
        capi.bump_counter(epoch)
        capi.push_rows_signal(rows, idx, send_ptr, [b.data_ptr() for b in bufs], first, dim, rank,
                              [w.data_ptr() for w in landed], epoch, done)
        torch.cuda.synchronize()
        assert epoch.item() == turn and not done.any().item()
        for r, c in enumerate(counts):
            want = rows[idx[send_ptr[r]:send_ptr[r + 1]].long()]
            assert torch.equal(bufs[r][first[r]:first[r] + c], want)
            assert bool((bufs[r][:first[r]] == -1).all()) and bool((bufs[r][first[r] + c:] == -1).all())
            assert landed[r][rank].item() == (turn if c else 0)
            assert int(landed[r].sum().item()) == (turn if c else 0)
        rows.mul_(2.0)


def test_wait_for_landed_rows_passes_and_gives_up(cuda):
    landed = torch.zeros(64, dtype=torch.int32, device=cuda)
    epoch = torch.full((1,), 3, dtype=torch.int32, device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    landed[2], landed[5] = 3, 4                                  # rank 5 is already one exchange ahead
    capi.wait_landed(landed, [2, 5], epoch, status, max_polls=2000)
    capi.wait_landed(landed, [], epoch, status, max_polls=2000)
    torch.cuda.synchronize()
    assert status.item() == capi.EPP_OK
    capi.wait_landed(landed, [2, 6], epoch, status, max_polls=2000)     # nothing from rank 6: the wait runs out
    torch.cuda.synchronize()
    assert status.item() == capi.EPP_ERR_PEER_TIMEOUT
    capi.wait_landed(landed, [6], epoch, status, max_polls=10_000_000)  # a broken group does not wait again
    torch.cuda.synchronize()
    assert status.item() == capi.EPP_ERR_PEER_TIMEOUT
