"""The compaction entry point that allocates nothing.

Some users of this library cannot allocate device memory while they run (their
own pool owns the whole GPU, or they cannot afford the synchronisation an
allocation implies), so ``eppgcn_compact_mask_static`` keeps its scan scratch in
a fixed array inside the library.  It must give exactly what the regular entry
point gives -- compaction is integer work, so the comparison is bit-exact -- and
because every call reuses the same array, it must do so twice in a row, the
second time on a different and smaller input than the first.

This file sorts last on purpose: a run that stops at the first failure has then
already executed every other test.
"""
import numpy as np
import pytest
import torch

from eppgcn_b200 import capi

pytestmark = pytest.mark.gpu


def make_case(length, keep, seed, dev):
    rng = np.random.Generator(np.random.PCG64(seed))
    mask = np.where(rng.random(length) < keep, rng.integers(0, 1 << 20, length), -1).astype(np.int32)
    col = rng.integers(0, 1 << 20, length).astype(np.int32)
    return torch.from_numpy(mask).to(dev), torch.from_numpy(col).to(dev)


def test_static_scratch_compaction_matches_regular_entry_point(cuda):
    # all buffers are made up front; the calls under test only receive pointers
    cases = [make_case(1_500_003, 0.6, 1, cuda), make_case(70_001, 0.1, 2, cuda)]
    outs = [(torch.full_like(m, 7), torch.full_like(c, 7)) for m, c in cases]
    counter = torch.empty(2, dtype=torch.int32, device=cuda)
    torch.cuda.synchronize()
    for (mask, col), (out_id, out_edge) in zip(cases, outs):         # two calls in a row, sharing the array
        valid = capi.compact_mask_static(mask, col, out_id, out_edge, counter)
        want_id, want_edge, want_valid = capi.compact_mask(mask, col)
        assert valid == want_valid
        assert torch.equal(out_id, want_id) and torch.equal(out_edge, want_edge)
        kept = mask != -1
        assert valid == int(kept.sum()) and torch.equal(out_id[:valid], mask[kept])


def test_a_call_after_the_warm_up_allocates_nothing(cuda):
    """After one warm-up call on the device, a call changes neither the free
    device memory the driver reports nor what torch's allocator holds: the
    caller's buffers and the built-in array are all it touches."""
    l = capi.lib()
    mask, col = make_case(300_001, 0.5, 4, cuda)
    out_id, out_edge = torch.empty_like(mask), torch.empty_like(col)
    counter = torch.empty(2, dtype=torch.int32, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        rc = l.eppgcn_compact_mask_static(mask.data_ptr(), col.data_ptr(), out_id.data_ptr(), out_edge.data_ptr(),
                                          mask.numel(), counter.data_ptr(), counter.data_ptr() + 4, stream)
        assert rc == capi.EPP_OK
        torch.cuda.synchronize()

    call()                                                   # warm-up: module load, address look-up
    free_before, _ = torch.cuda.mem_get_info(cuda)
    held_before, reserved_before = torch.cuda.memory_allocated(cuda), torch.cuda.memory_reserved(cuda)
    for _ in range(2):
        call()
    free_after, _ = torch.cuda.mem_get_info(cuda)
    assert free_after == free_before, "free device memory changed across a call"
    assert torch.cuda.memory_allocated(cuda) == held_before and torch.cuda.memory_reserved(cuda) == reserved_before
    assert int(counter[1].item()) == capi.EPP_OK and int(counter[0].item()) == int((mask != -1).sum().item())


def test_static_scratch_edge_cases(cuda):
    counter = torch.empty(2, dtype=torch.int32, device=cuda)
    empty = torch.zeros(0, dtype=torch.int32, device=cuda)
    assert capi.compact_mask_static(empty, empty, empty, empty, counter) == 0
    mask, col = make_case(4097, 1.0, 3, cuda)                         # one full tile plus one element, all kept
    out_id, out_edge = torch.empty_like(mask), torch.empty_like(col)
    assert capi.compact_mask_static(mask, col, out_id, out_edge, counter) == 4097
    assert torch.equal(out_id, mask) and torch.equal(out_edge, col)


def test_static_scratch_rejects_oversize_input():
    """Beyond 2**26 edges the entry point refuses before touching the device
    (the length check comes first, so null pointers are never read)."""
    l = capi.lib()
    rc = l.eppgcn_compact_mask_static(None, None, None, None, (1 << 26) + 1, 8, 8, None)
    assert rc == capi.EPP_ERR_TOO_LARGE
    assert b"at most" in l.eppgcn_last_error()
