"""World-size-2 CPU test of the sharded path: two gloo ranks take their (batch x value-head)
shards, run the checker on their slice with global dropout coordinates, gather, and must
reproduce the unsharded result bit for bit; timings reduce with MAX over ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, batch, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import rosa_oracle as orc
        from rosa_soft_b200 import sharding

        B, T, H, D, Hv, Dv, W = batch, 24, 4, 3, 2, 3, 5
        g = torch.Generator().manual_seed(3)
        q, k = torch.randn(B, T, H, D, generator=g), torch.randn(B, T, H, D, generator=g)
        v, go = torch.randn(B, T, Hv, Dv, generator=g), torch.randn(B, T, H, Dv, generator=g)
        group = H // Hv
        sh = sharding.shard_dense(B, Hv, world, rank)
        bs = slice(sh.batch_start, sh.batch_stop)
        hs, vs = sh.head_slice(group), slice(sh.value_head_start, sh.value_head_stop)
        nb = sh.batch_stop - sh.batch_start
        flat = lambda t: np.ascontiguousarray(t.numpy()).reshape((nb * T,) + tuple(t.shape[2:]))
        cu = np.arange(nb + 1, dtype=np.int64) * T
        dq, dk, dv = orc.surrogate_vjp(flat(q[bs][:, :, hs]), flat(k[bs][:, :, hs]),
                                       flat(v[bs][:, :, vs]), flat(go[bs][:, :, hs]), cu, W, 1.0,
                                       0.3, 3.0, seed=99, batch_offset=sh.dropout_batch_offset,
                                       head_offset=sh.dropout_head_offset(group))
        mine = torch.from_numpy(dq).reshape(nb, T, hs.stop - hs.start, D)
        gathered = sharding.gather_along(mine, 0 if world <= B else 2)
        slowest = sharding.max_over_ranks(10.0 + rank)
        if rank == 0:
            cu_all = np.arange(B + 1, dtype=np.int64) * T
            fl = lambda t: t.numpy().reshape((B * T,) + tuple(t.shape[2:]))
            full, _, _ = orc.surrogate_vjp(fl(q), fl(k), fl(v), fl(go), cu_all, W, 1.0, 0.3, 3.0,
                                           seed=99)
            results["equal"] = bool(np.array_equal(gathered.numpy().reshape(full.shape), full))
            results["slowest"] = slowest
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("batch", [2, 1])   # split by batch, then by value-head group
def test_two_rank_shards_reproduce_the_unsharded_gradients(batch):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, _free_port(), batch, results), nprocs=2, join=True)
    assert results["equal"] is True
    assert results["slowest"] == 11.0


def test_shard_bookkeeping():
    from rosa_soft_b200 import sharding

    units = set()
    for rank in range(8):
        sh = sharding.shard_dense(2, 16, 8, rank)
        for b in range(sh.batch_start, sh.batch_stop):
            for vh in range(sh.value_head_start, sh.value_head_stop):
                assert (b, vh) not in units
                units.add((b, vh))
        assert sh.dropout_head_offset(4) == sh.value_head_start * 4
    assert len(units) == 32
    assert sharding.shard_dense(8, 3, 4, 1) == sharding.DenseShard(2, 4, 0, 3)
    with pytest.raises(ValueError):
        sharding.shard_dense(3, 4, 2, 0)
    owned = sharding.balance_sequences([4096, 64, 3000, 3000, 100, 2048], 2)
    assert sorted(sum(owned, [])) == list(range(6))
    loads = [sum(l * l for l in ([4096, 64, 3000, 3000, 100, 2048][s] for s in o)) for o in owned]
    assert max(loads) / min(loads) < 1.3


def test_packed_shards_keep_every_sequence_ordinal():
    """A rank's cu_seqlens names all sequences (foreign ones empty), so the sequence ordinal --
    the dropout counter's batch word for packed batches -- needs no offset: the oracle on the
    two shares reproduces the unsharded packed gradients bit for bit."""
    from oracle import rosa_oracle as orc
    from rosa_soft_b200 import sharding

    lengths = [20, 0, 33, 5, 27]
    N, H, D, Hv, Dv, W = sum(lengths), 2, 3, 1, 4, 6
    rng = np.random.default_rng(4)
    q, k = rng.standard_normal((N, H, D)), rng.standard_normal((N, H, D))
    v, go = rng.standard_normal((N, Hv, Dv)), rng.standard_normal((N, H, Dv))
    cu_full = np.concatenate([[0], np.cumsum(lengths)])
    full = orc.surrogate_vjp(q, k, v, go, cu_full, W, 1.0, 0.4, 3.0, seed=5)
    owned = sharding.balance_sequences(lengths, 2)
    seen = np.zeros(N, bool)
    for rank in range(2):
        cu, ranges = sharding.packed_shard_offsets(lengths, owned[rank])
        assert len(cu) == len(lengths) + 1 and cu[-1] == sum(lengths[s] for s in owned[rank])
        idx = np.concatenate([np.arange(a, b) for a, b in ranges])
        assert not seen[idx].any()
        seen[idx] = True
        part = orc.surrogate_vjp(q[idx], k[idx], v[idx], go[idx], np.array(cu), W, 1.0, 0.4, 3.0,
                                 seed=5)
        for mine, want in zip(part, full):
            assert np.array_equal(mine, want[idx])
    assert seen.all()
    with sharding.dropout_coordinates(3, 8):
        assert sharding.current_dropout_coordinates() == (3, 8)
    assert sharding.current_dropout_coordinates() == (0, 0)
