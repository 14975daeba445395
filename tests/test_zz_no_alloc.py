"""The workspace-free hard forward (rosa_b200_hard_forward_static).

Some hosts cannot hand the library a scratch buffer: they gave all device memory to their
own arena, or they have no device allocator at all.  For them the library keeps a fixed
scratch array in its own device image.  This file checks, through the C ABI, that the
static variant returns exactly what the workspace variant returns -- on two calls in a row
with different problems, because the shared array still holds the first call's data when
the second one starts -- that the call leaves the amount of free device memory unchanged, that
a bad offsets array is reported through the status path that needs no workspace pointer, that
the largest problem it accepts stays inside the array, and that larger ones are refused.
It is named to be collected last so that a failure here cannot hide another test."""
import numpy as np
import pytest
import torch

from tests.helpers import nonzero_randn, repeated_stream_logits

DEV = "cuda"


def _pair(cabi, q, k, v, desc, W):
    ref = cabi.hard_forward(q, k, v, desc, W)[:4]
    got = cabi.hard_forward_static(q, k, v, desc, W)
    torch.cuda.synchronize()
    for a, b in zip(got, ref):
        assert torch.equal(a, b)


@pytest.mark.gpu
def test_static_variant_matches_workspace_variant_twice_in_a_row():
    from rosa_soft_b200 import cabi
    cabi.load()
    # first call: long repeated matches over two dense sequences (many rows find a winner)
    B, T, H, D, Hv, Dv = 2, 1500, 4, 2, 2, 6
    q = repeated_stream_logits(B * T, H, D, seed=21).to(DEV)
    v = nonzero_randn((B * T, Hv, Dv), 22).to(DEV)
    _pair(cabi, q, q.clone(), v, (B, T), 64)
    # second call: a smaller packed problem with few matches; stale winners from the first
    # call would show up as wrong routes here
    lengths = [7, 0, 400, 1, 93]
    N = sum(lengths)
    cu = torch.tensor([0, 7, 7, 407, 408, 501], dtype=torch.int32, device=DEV)
    q2 = nonzero_randn((N, 2, 9), 23, torch.bfloat16).to(DEV)
    k2 = nonzero_randn((N, 2, 9), 24, torch.bfloat16).to(DEV)
    v2 = nonzero_randn((N, 1, 5), 25, torch.bfloat16).to(DEV)
    _pair(cabi, q2, k2, v2, cu, 16)
    # and the first problem again
    _pair(cabi, q, q.clone(), v, (B, T), 64)


@pytest.mark.gpu
def test_static_variant_leaves_free_device_memory_unchanged():
    """The point of the entry point: between two calls (the first one has resolved the array's
    address) the driver reports the same amount of free memory, and so does torch's allocator
    for everything but the output tensors the test itself passes in."""
    import ctypes
    from rosa_soft_b200 import cabi
    lib = cabi.load()
    N, H, D, Hv, Dv, W = 3000, 4, 3, 2, 4, 32
    q = repeated_stream_logits(N, H, D, seed=31).to(DEV)
    v = nonzero_randn((N, Hv, Dv), 32).to(DEV)
    out = torch.empty((N, H, Dv), device=DEV)
    pq = torch.empty((1, H, N), dtype=torch.int32, device=DEV)
    pk = torch.empty_like(pq)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call():
        rc = lib.rosa_b200_hard_forward_static(ptr(q), ptr(q), ptr(v), cabi.F32, N, H, D, Hv, Dv,
                                               None, 1, N, W, ptr(out), ptr(pq), ptr(pk), None, stream)
        assert rc == 0, cabi.last_error()

    call()                                   # resolves the scratch address on this device
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    call()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.cuda.memory_reserved() == reserved_before
    ref = cabi.hard_forward(q, q, v, (1, N), W)[0]
    assert torch.equal(out, ref)


@pytest.mark.gpu
def test_static_variant_reports_bad_offsets_without_a_workspace_pointer():
    """Inconsistent cu_seqlens: every kernel of the call is a no-op (outputs zero, routes -1) and
    rosa_b200_read_status(NULL, ...) returns the code; a good call afterwards clears it."""
    from rosa_soft_b200 import cabi
    cabi.load()
    N, H, D, Dv = 20, 2, 3, 4
    q = nonzero_randn((N, H, D), 71).to(DEV)
    v = nonzero_randn((N, 1, Dv), 72).to(DEV)
    for offsets, status in (([1, 10, 20], 1), ([0, 12, 8, 20], 2), ([0, 10, 19], 3)):
        cu = torch.tensor(offsets, dtype=torch.int32, device=DEV)
        out, pq, pk, routes = cabi.hard_forward_static(q, q, v, cu, 8)
        assert cabi.read_status(None) == status
        assert not out.any() and torch.all(routes == -1)
    cu = torch.tensor([0, 10, 20], dtype=torch.int32, device=DEV)
    out, pq, pk, routes = cabi.hard_forward_static(q, q, v, cu, 8)
    assert cabi.read_status(None) == 0
    assert torch.equal(out, cabi.hard_forward(q, q, v, cu, 8)[0])


@pytest.mark.gpu
def test_static_variant_at_its_capacity_limits():
    """Exactly 1,048,576 token-heads in exactly 4096 packed sequences (empty ones included): the
    plan tables and the winner table fill the array to its last byte.  Bit-equal to the workspace
    variant, and a small call afterwards still works (nothing beyond the array was needed)."""
    from rosa_soft_b200 import cabi
    cabi.load()
    H, S = 4, 4096
    N = (1 << 20) // H
    rng = np.random.default_rng(5)
    cuts = np.sort(rng.integers(0, N + 1, size=S - 1))
    cuts[100:140] = cuts[100]                # a run of empty sequences
    cu_np = np.concatenate([[0], np.sort(cuts), [N]]).astype(np.int32)
    cu = torch.from_numpy(cu_np).to(DEV)
    q = repeated_stream_logits(N, H, 2, seed=77, seg=(4, 24)).to(DEV)
    v = nonzero_randn((N, 2, 3), 78).to(DEV)
    _pair(cabi, q, q.clone(), v, cu, 16)
    assert cabi.read_status(None) == 0
    small_q = nonzero_randn((50, 1, 2), 79).to(DEV)
    _pair(cabi, small_q, small_q.clone(), nonzero_randn((50, 1, 2), 80).to(DEV), (1, 50), 4)


def test_static_variant_rejects_problems_beyond_its_capacity():
    from rosa_soft_b200 import cabi
    lib = cabi.load()
    one = 1  # non-null dummies: the size check comes before any pointer is used
    rc = lib.rosa_b200_hard_forward_static(one, one, one, 0, (1 << 20) + 2, 2, 4, 1, 4, None, 1,
                                           (1 << 20) + 2, 8, one, one, one, None, None)
    assert rc != 0 and "at most 1048576 token-heads" in cabi.last_error()
    rc = lib.rosa_b200_hard_forward_static(one, one, one, 0, 8192, 1, 4, 1, 4, one, 5000, 0, 8, one,
                                           one, one, None, None)
    assert rc != 0 and "at most 4096 sequences" in cabi.last_error()
