"""A fixed problem split over two GPUs equals the one-GPU run bit for bit.

Each rank runs the public operator on its share -- (batch x value-head group) units of a dense
batch, whole sequences of a packed batch with every ordinal kept -- inside
`sharding.dropout_coordinates`, gathers outputs and gradients over NCCL and compares them with
the unsharded run it computes itself.  Needs two CUDA devices; skipped otherwise."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, failures):
    import torch.distributed as dist

    import rosa_soft_b200 as rs
    from rosa_soft_b200 import sharding
    from tests.helpers import nonzero_randn

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        kw = dict(max_suffix_length=24, scale=1.0, dropout_p=0.2, mismatch_scale=3.0)

        def run(q, k, v, go, cu=None, offsets=(0, 0)):
            q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
            torch.cuda.manual_seed(77)               # same dropout seed on every rank
            with sharding.dropout_coordinates(*offsets):
                out = rs.rosa_soft(q, k, v, **kw) if cu is None else rs.rosa_soft_varlen(q, k, v, cu, **kw)
                out.backward(go)
            return out.detach(), q.grad, k.grad, v.grad

        # ---- dense: B=2, Hv=2 over 2 ranks by batch, then B=1 over 2 ranks by value head
        for B, T, H, D, Hv, Dv in ((2, 300, 4, 4, 2, 8), (1, 280, 4, 3, 2, 12)):
            q = nonzero_randn((B, T, H, D), 1).to(dev)
            k = nonzero_randn((B, T, H, D), 2).to(dev)
            v = nonzero_randn((B, T, Hv, Dv), 3).to(dev)
            go = nonzero_randn((B, T, H, Dv), 4).to(dev)
            full = run(q, k, v, go)
            shard = sharding.shard_dense(B, Hv, world, rank)
            group = H // Hv
            bs = slice(shard.batch_start, shard.batch_stop)
            hs = shard.head_slice(group)
            vs = slice(shard.value_head_start, shard.value_head_stop)
            mine = run(q[bs, :, hs].contiguous(), k[bs, :, hs].contiguous(), v[bs, :, vs].contiguous(),
                       go[bs, :, hs].contiguous(),
                       offsets=(shard.dropout_batch_offset, shard.dropout_head_offset(group)))
            dim = 0 if world <= B else 2
            for got, want in zip(mine, full):
                gathered = sharding.gather_along(got, dim)
                if not torch.equal(gathered, want):
                    failures.put((rank, "dense", B, tuple(got.shape)))
        # ---- packed: sequences assigned by squared length, every ordinal kept
        lengths = [90, 0, 310, 5, 200, 64]
        N, H, D, Hv, Dv = sum(lengths), 2, 5, 1, 6
        q = nonzero_randn((N, H, D), 11).to(dev)
        k = nonzero_randn((N, H, D), 12).to(dev)
        v = nonzero_randn((N, Hv, Dv), 13).to(dev)
        go = nonzero_randn((N, H, Dv), 14).to(dev)
        cu_full = torch.tensor([0] + list(__import__("itertools").accumulate(lengths)),
                               dtype=torch.int32, device=dev)
        full = run(q, k, v, go, cu_full)
        owned = sharding.balance_sequences(lengths, world)
        cu_list, ranges = sharding.packed_shard_offsets(lengths, owned[rank])
        take = lambda t: torch.cat([t[a:b] for a, b in ranges], 0).contiguous()
        mine = run(take(q), take(k), take(v), take(go),
                   torch.tensor(cu_list, dtype=torch.int32, device=dev))
        for got, want in zip(mine, full):
            if not torch.equal(got, take(want)):
                failures.put((rank, "packed", tuple(got.shape)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_shards_equal_the_unsharded_run():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    mp.spawn(_worker, args=(2, _free_port(), failures), nprocs=2, join=True)
    problems = []
    while not failures.empty():
        problems.append(failures.get())
    assert not problems, problems
