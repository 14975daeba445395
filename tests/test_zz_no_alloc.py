"""The workspace-free hard forward (rosa_b200_hard_forward_static).

Some hosts cannot hand the library a scratch buffer: they gave all device memory to their
own arena, or they have no device allocator at all.  For them the library keeps a fixed
scratch array in its own device image.  This file checks, through the C ABI, that the
static variant returns exactly what the workspace variant returns -- on two calls in a row
with different problems, because the shared array still holds the first call's data when
the second one starts -- and that problems beyond the array's capacity are refused.
It is named to be collected last so that a failure here cannot hide another test."""
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


def test_static_variant_rejects_problems_beyond_its_capacity():
    from rosa_soft_b200 import cabi
    lib = cabi.load()
    one = 1  # non-null dummies: the size check comes before any pointer is used
    rc = lib.rosa_b200_hard_forward_static(one, one, one, 0, 1 << 20, 2, 4, 1, 4, None, 1, 1 << 20,
                                           8, one, one, one, None, None)
    assert rc != 0 and "at most 1048576 token-heads" in cabi.last_error()
    rc = lib.rosa_b200_hard_forward_static(one, one, one, 0, 8192, 1, 4, 1, 4, one, 5000, 0, 8, one,
                                           one, one, None, None)
    assert rc != 0 and "at most 4096 sequences" in cabi.last_error()
