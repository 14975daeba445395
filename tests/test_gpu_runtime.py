"""GPU streaming runtime (rosa_soft_b200.RosaRuntime) against the CPU oracle and the outputs of
the reference's own RosaRuntime (fixture runtime_cases): any chunking of a stream must give the
one-shot result (reference tests/test_runtime.py:271-317), slots are fixed by the first update,
reset starts over, the state survives a state_dict round trip."""
import os

import numpy as np
import pytest
import torch

from oracle import rosa_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _symbols(shape, bits, seed, repeat=0.0):
    rng = np.random.default_rng(seed)
    x = rng.integers(0, 1 << bits, size=shape, dtype=np.uint8)
    if repeat > 0.0:   # copy earlier stretches forward so that long matches exist
        flat = x.reshape(-1, shape[-1]) if len(shape) == 2 else x
        n = flat.shape[-2]
        for _ in range(max(1, int(repeat * n / 16))):
            length = int(rng.integers(4, 48))
            if n <= 2 * length:
                continue
            src = int(rng.integers(0, n - 2 * length))
            dst = int(rng.integers(src + length, n - length))
            flat[..., dst:dst + length, :] = flat[..., src:src + length, :]
    return x


def _oracle_streams(q, k, p, lengths, W):
    """q, k [N, H] uint8, p [N, Hp] uint8 packed by stream -> (out uint8 [N, H], end int64)."""
    cu = np.concatenate([[0], np.cumsum(lengths)])
    out, end = orc.hard_inference(q.astype(np.uint32), k.astype(np.uint32),
                                  p.astype(np.float32)[:, :, None], cu, W)
    return out[:, :, 0].astype(np.uint8), end


def _run_chunked(rt, q, k, p, lengths, cuts):
    """Feeds streams (packed one after another in q/k/p) in rounds; round r gives slot s the
    tokens [cuts[s][r], cuts[s][r+1]).  Returns the per-stream concatenation of the results."""
    starts = np.concatenate([[0], np.cumsum(lengths)])[:-1]
    rounds = len(cuts[0]) - 1
    outs = [[] for _ in lengths]
    ends = [[] for _ in lengths]
    for r in range(rounds):
        idx = [np.arange(starts[s] + cuts[s][r], starts[s] + cuts[s][r + 1]) for s in range(len(lengths))]
        cu = np.concatenate([[0], np.cumsum([len(i) for i in idx])])
        sel = np.concatenate(idx).astype(np.int64)
        out, end = rt.update_packed(torch.from_numpy(q[sel]).to(DEV), torch.from_numpy(k[sel]).to(DEV),
                                    torch.from_numpy(p[sel]).to(DEV),
                                    cu_seqlens=torch.from_numpy(cu.astype(np.int32)).to(DEV))
        out, end = out.cpu().numpy(), end.cpu().numpy()
        for s in range(len(lengths)):
            outs[s].append(out[cu[s]:cu[s + 1]])
            ends[s].append(end[cu[s]:cu[s + 1]])
    return (np.concatenate([np.concatenate(o) for o in outs]),
            np.concatenate([np.concatenate(e) for e in ends]))


def test_chunked_dense_updates_equal_one_shot_and_oracle():
    from rosa_soft_b200 import RosaRuntime
    B, T, H, Hp, bits, W = 2, 24, 4, 2, 3, 5
    q, k, p = (_symbols((B, T, n), bits, seed) for n, seed in ((H, 7), (H, 8), (Hp, 9)))
    want_out, want_end = _oracle_streams(q.reshape(-1, H), k.reshape(-1, H), p.reshape(-1, Hp), [T] * B, W)
    tq, tk, tp = (torch.from_numpy(x).to(DEV) for x in (q, k, p))
    with RosaRuntime(H, Hp, bits, bits, W) as one_shot:
        out, end = one_shot.update_packed(tq, tk, tp)
    assert out.dtype == torch.uint8 and end.dtype == torch.int64 and out.shape == (B, T, H)
    assert np.array_equal(out.cpu().numpy().reshape(-1, H), want_out)
    assert np.array_equal(end.cpu().numpy().reshape(-1, H), want_end)
    cuts = [0, 3, 11, 17, T]
    outs, ends = [], []
    with RosaRuntime(H, Hp, bits, bits, W) as chunked:
        for a, b in zip(cuts[:-1], cuts[1:]):
            o, e = chunked.update_packed(tq[:, a:b], tk[:, a:b], tp[:, a:b])
            outs.append(o)
            ends.append(e)
    assert torch.equal(torch.cat(outs, dim=1), out)
    assert torch.equal(torch.cat(ends, dim=1), end)


@pytest.mark.parametrize("W,bits,lengths", [
    (1, 1, (40, 1, 0, 300)),
    (32, 2, (700, 513, 64)),          # crosses the first capacity (256) twice
    (300, 1, (1200, 5)),
    (7, 8, (90, 257, 31, 2)),
])
def test_ragged_chunks_with_empty_slots_match_oracle(W, bits, lengths):
    from rosa_soft_b200 import RosaRuntime
    H, Hp = 4, 2
    N = sum(lengths)
    q, k, p = (_symbols((N, n), bits, seed, repeat=0.5) for n, seed in ((H, 1), (H, 2), (Hp, 3)))
    k[:] = np.where(np.random.default_rng(4).random(k.shape) < 0.7, q, k)   # q often equals k
    want_out, want_end = _oracle_streams(q, k, p, lengths, W)
    rng = np.random.default_rng(5)
    rounds = 6
    cuts = []
    for L in lengths:
        inner = np.sort(rng.integers(0, L + 1, size=rounds - 1))
        cuts.append([0, *inner.tolist(), L])
    rt = RosaRuntime(H, Hp, bits, 8, W)
    got_out, got_end = _run_chunked(rt, q, k, p, lengths, cuts)
    assert np.array_equal(got_end, want_end)
    assert np.array_equal(got_out, want_out)
    stats = rt.memory_stats()
    assert stats["sequences"] == len(lengths) and stats["payload_symbols"] == N * Hp
    rt.close()
    assert rt.state == "CLOSED"
    with pytest.raises(RuntimeError, match="closed"):
        rt.update_packed(torch.zeros((1, 1, H), dtype=torch.uint8, device=DEV),
                         torch.zeros((1, 1, H), dtype=torch.uint8, device=DEV),
                         torch.zeros((1, 1, Hp), dtype=torch.uint8, device=DEV))


def test_reference_runtime_fixture_in_chunks():
    from rosa_soft_b200 import RosaRuntime
    z = np.load(os.path.join(GOLDEN, "runtime_cases.npz"))
    for c in range(int(z["n"])):
        cu, W = z[f"c{c}_cu"], int(z[f"c{c}_W"])
        q, k, p = z[f"c{c}_q"], z[f"c{c}_k"], z[f"c{c}_payload"]
        lengths = np.diff(cu).tolist()
        rng = np.random.default_rng(c)
        cuts = [[0, *np.sort(rng.integers(0, L + 1, size=3)).tolist(), L] for L in lengths]
        rt = RosaRuntime(q.shape[1], p.shape[1], 8, 8, W)
        got_out, got_end = _run_chunked(rt, q, k, p, lengths, cuts)
        assert np.array_equal(got_end, z[f"c{c}_end"]), c
        assert np.array_equal(got_out, z[f"c{c}_out"]), c


def test_token_by_token_decode_after_prefill():
    from rosa_soft_b200 import RosaRuntime
    H, Hp, bits, W, L, steps = 8, 4, 2, 16, 1000, 40
    lengths = [L + steps, L + steps]
    N = sum(lengths)
    q, k, p = (_symbols((N, n), bits, seed, repeat=0.5) for n, seed in ((H, 11), (H, 12), (Hp, 13)))
    want_out, want_end = _oracle_streams(q, k, p, lengths, W)
    cuts = [[0, L, *range(L + 1, L + steps + 1)] for _ in lengths]
    rt = RosaRuntime(H, Hp, bits, bits, W)
    got_out, got_end = _run_chunked(rt, q, k, p, lengths, cuts)
    assert np.array_equal(got_end, want_end) and np.array_equal(got_out, want_out)


def test_wide_keys_for_long_horizons():
    """A horizon of thousands of tokens on a nearly constant stream: the match lengths reach the
    horizon, the level loop of the bit matcher runs thousands of steps per word."""
    from rosa_soft_b200 import RosaRuntime
    H, Hp, W, L = 2, 1, 3000, 3500
    q = np.zeros((L, H), dtype=np.uint8)
    q[::977, 1] = 1
    k = q.copy()
    p = _symbols((L, Hp), 8, 21)
    want_out, want_end = _oracle_streams(q, k, p, [L], W)
    rt = RosaRuntime(H, Hp, 1, 8, W)
    got_out, got_end = _run_chunked(rt, q, k, p, [L], [[0, 1700, 1701, L]])
    assert np.array_equal(got_end, want_end) and np.array_equal(got_out, want_out)


def test_update_from_logits_unpacks_and_masks_null_rows():
    from rosa_soft_b200 import RosaRuntime
    from rosa_soft_b200.runtime import pack_sign_bits
    B, T, H, Hp, qb, pb, W = 2, 50, 4, 2, 3, 5, 8
    g = torch.Generator().manual_seed(3)
    ql = torch.randn(B, T, H, qb, generator=g).to(DEV)
    kl = torch.where(torch.rand(B, T, H, qb, generator=g).to(DEV) < 0.8, ql, -ql)
    pl = torch.randn(B, T, Hp, pb, generator=g).to(DEV).to(torch.bfloat16)
    rt = RosaRuntime(H, Hp, qb, pb, W)
    values, end = rt.update(ql, kl, pl)
    assert values.shape == (B, T, H, pb) and values.dtype == torch.bfloat16
    rt.reset()
    packed, end2 = rt.update_packed(pack_sign_bits(ql), pack_sign_bits(kl), pack_sign_bits(pl))
    assert torch.equal(end, end2)
    null = end < 0
    assert null[:, 0].all() and torch.all(values[null] == 0)
    hit = ~null
    bits = ((packed[hit].to(torch.int32).unsqueeze(-1) >> torch.arange(pb, device=DEV)) & 1) * 2 - 1
    assert torch.equal(values[hit].float(), bits.float())
    # the successor payload really is the stored one
    b, t, h = (x[0].item() for x in torch.nonzero(hit, as_tuple=True))
    succ = end[b, t, h].item() + 1
    assert packed[b, t, h].item() == pack_sign_bits(pl)[b, succ, h // (H // Hp)].item()


def test_slots_sequence_ids_reset_and_state_dict():
    from rosa_soft_b200 import RosaRuntime
    H, Hp, bits, W = 2, 2, 2, 4
    mk = lambda B, T, n, seed: torch.from_numpy(_symbols((B, T, n), bits, seed)).to(DEV)
    rt = RosaRuntime(H, Hp, bits, bits, W)
    rt.update_packed(mk(3, 5, H, 1), mk(3, 5, H, 2), mk(3, 5, Hp, 3), sequence_ids=[10, 11, 12])
    with pytest.raises(RuntimeError, match="slot count is fixed"):
        rt.update_packed(mk(2, 5, H, 1), mk(2, 5, H, 2), mk(2, 5, Hp, 3), sequence_ids=[10, 11])
    with pytest.raises(RuntimeError, match="sequence_ids changed"):
        rt.update_packed(mk(3, 5, H, 1), mk(3, 5, H, 2), mk(3, 5, Hp, 3), sequence_ids=[11, 10, 12])
    with pytest.raises(RuntimeError, match="sequence_ids are required"):
        rt.update_packed(mk(3, 5, H, 1), mk(3, 5, H, 2), mk(3, 5, Hp, 3))
    with pytest.raises(ValueError, match="unique"):
        rt.update_packed(mk(3, 5, H, 1), mk(3, 5, H, 2), mk(3, 5, Hp, 3), sequence_ids=[1, 1, 2])
    # a failed check leaves the streams where they were: resume and compare with a fresh run
    q2, k2, p2 = mk(3, 7, H, 4), mk(3, 7, H, 5), mk(3, 7, Hp, 6)
    saved = rt.state_dict()
    out_a, end_a = rt.update_packed(q2, k2, p2, sequence_ids=[10, 11, 12])
    other = RosaRuntime(H, Hp, bits, bits, W)
    other.load_state_dict(saved)
    out_b, end_b = other.update_packed(q2, k2, p2, sequence_ids=[10, 11, 12])
    assert torch.equal(out_a, out_b) and torch.equal(end_a, end_b)
    fresh = RosaRuntime(H, Hp, bits, bits, W)
    full_q = torch.cat([mk(3, 5, H, 1), q2], dim=1)
    full_k = torch.cat([mk(3, 5, H, 2), k2], dim=1)
    full_p = torch.cat([mk(3, 5, Hp, 3), p2], dim=1)
    out_f, end_f = fresh.update_packed(full_q, full_k, full_p)
    assert torch.equal(out_f[:, 5:], out_a) and torch.equal(end_f[:, 5:], end_a)
    # reset forgets slots and ids
    rt.reset()
    out_r, end_r = rt.update_packed(full_q[:2], full_k[:2], full_p[:2])
    assert torch.equal(out_r, out_f[:2]) and torch.equal(end_r, end_f[:2])


def test_side_stream_and_async_handle():
    from rosa_soft_b200 import RosaRuntime
    H, Hp, bits, W = 4, 4, 3, 6
    mk = lambda T, n, seed: torch.from_numpy(_symbols((2, T, n), bits, seed)).to(DEV)
    q, k, p = mk(300, H, 1), mk(300, H, 2), mk(300, Hp, 3)
    base = RosaRuntime(H, Hp, bits, bits, W).update_packed(q, k, p)
    side = torch.cuda.Stream()
    rt = RosaRuntime(H, Hp, bits, bits, W)
    work = rt.update_packed(q[:, :100], k[:, :100], p[:, :100], stream=side, async_op=True)
    first = work.wait()
    second = rt.update_packed(q[:, 100:], k[:, 100:], p[:, 100:], stream=side)
    torch.cuda.synchronize()
    assert torch.equal(torch.cat([first[0], second[0]], dim=1), base[0])
    assert torch.equal(torch.cat([first[1], second[1]], dim=1), base[1])


def test_c_abi_reports_capacity_and_bad_offsets_without_touching_state():
    from rosa_soft_b200 import cabi
    S, H, Hp, cap, bits = 2, 2, 1, 64, 1
    km = torch.zeros((S, H, 1 << bits, cap // 32), dtype=torch.int32, device=DEV)
    qh = torch.zeros((S, H, cap), dtype=torch.uint8, device=DEV)
    ph = torch.zeros((S, Hp, cap), dtype=torch.uint8, device=DEV)
    lengths = torch.tensor([60, 3], dtype=torch.int32, device=DEV)
    n = 10
    q = torch.ones((n, H), dtype=torch.uint8, device=DEV)
    p = torch.ones((n, Hp), dtype=torch.uint8, device=DEV)
    off = torch.tensor([0, 5, 10], dtype=torch.int32, device=DEV)      # slot 0 would reach 65 > 64
    _, _, ws = cabi.stream_update(q, q, p, off, bits, 1, 4, km, qh, ph, lengths, 64)
    assert cabi.read_status(ws) == 4
    assert lengths.tolist() == [60, 3] and int(km.ne(0).sum()) == 0 and int(qh.sum()) == 0
    off = torch.tensor([0, 3, 2], dtype=torch.int32, device=DEV)
    _, _, ws = cabi.stream_update(q, q, p, off, bits, 1, 4, km, qh, ph, lengths, 64)
    assert cabi.read_status(ws) in (2, 3)
    assert lengths.tolist() == [60, 3]
    off = torch.tensor([0, 4, 10], dtype=torch.int32, device=DEV)
    _, _, ws = cabi.stream_update(q, q, p, off, bits, 1, 4, km, qh, ph, lengths, 64)
    assert cabi.read_status(ws) == 0
    assert lengths.tolist() == [64, 9]
    # the appended key symbols (all 1) are bits 60..63 of slot 0 and 3..8 of slot 1 in bitmap 1
    words = km.view(S, H, 2, cap // 32).cpu().numpy().astype("uint32")
    assert int(words[0, 0, 1, 1]) == 0xF0000000 and int(words[1, 1, 1, 0]) == 0x1F8
    assert int(words[:, :, 0].sum()) == 0


def test_updates_on_different_streams_are_ordered_and_empty_first_update_works():
    """The state is shared by all updates: an update on an explicit stream followed by one on
    another stream must see the first one's appended tokens; a first update without tokens is
    accepted (the reference accepts zero-token updates)."""
    from rosa_soft_b200 import RosaRuntime
    H, Hp, bits, W, T = 3, 1, 3, 12, 700
    q = _symbols((T, H), bits, 91, repeat=0.4)
    k = _symbols((T, H), bits, 92, repeat=0.4)
    p = _symbols((T, Hp), 8, 93)
    want_out, want_end = _oracle_streams(q, k, p, [T], W)
    rt = RosaRuntime(H, Hp, bits, 8, W)
    empty = torch.zeros((0, H), dtype=torch.uint8, device=DEV)
    out0, end0 = rt.update_packed(empty, empty, torch.zeros((0, Hp), dtype=torch.uint8, device=DEV),
                                  cu_seqlens=torch.tensor([0, 0], dtype=torch.int32, device=DEV))
    assert out0.shape == (0, H) and end0.shape == (0, H)
    streams = [torch.cuda.Stream(), torch.cuda.Stream(), None]
    outs, ends, works = [], [], []
    cuts = [0, 300, 301, T]
    dev = lambda a: torch.from_numpy(a).to(DEV)
    for (a, b), st in zip(zip(cuts[:-1], cuts[1:]), streams):
        cu = torch.tensor([0, b - a], dtype=torch.int32, device=DEV)
        works.append(rt.update_packed(dev(q[a:b]), dev(k[a:b]), dev(p[a:b]), cu_seqlens=cu, stream=st,
                                      async_op=st is not None))
    for w in works:
        out, end = w.wait() if hasattr(w, "wait") else w
        outs.append(out)
        ends.append(end)
    torch.cuda.synchronize()
    assert np.array_equal(torch.cat(outs).cpu().numpy(), want_out)
    assert np.array_equal(torch.cat(ends).cpu().numpy(), want_end)


def test_custom_class_matches_the_python_runtime_and_the_reference_fixture():
    """torch.classes.rosa_soft.RosaRuntime (constructor and methods of the reference's class,
    rosa_soft/csrc/rosa_runtime.cpp:570-582) over the same streaming entry point."""
    import rosa_soft_b200  # noqa: F401  (registers the class)
    z = np.load(os.path.join(GOLDEN, "runtime_cases.npz"))
    H, Hp, bits, W = z["c1_q"].shape[1], z["c1_payload"].shape[1], 2, int(z["c1_W"])
    rt = torch.classes.rosa_soft.RosaRuntime(H, Hp, bits, 8, W)
    cu = torch.from_numpy(z["c1_cu"])            # int64 on the host, like the reference takes it
    out, end = rt.update_packed(cu, torch.from_numpy(z["c1_q"]).to(DEV),
                                torch.from_numpy(z["c1_k"]).to(DEV),
                                torch.from_numpy(z["c1_payload"]).to(DEV))
    assert np.array_equal(out.cpu().numpy(), z["c1_out"])
    assert np.array_equal(end.cpu().numpy(), z["c1_end"])
    states, edges, payload_symbols, automata, sequences, logical = rt.stats()
    slots = len(z["c1_cu"]) - 1
    assert (states, edges, automata, sequences) == (0, 0, slots * H, slots)
    assert payload_symbols == int(z["c1_cu"][-1]) * Hp and logical > 0
    with pytest.raises(RuntimeError, match="slot count is fixed"):
        rt.update_packed(cu[:2].clone(), torch.zeros((int(cu[1]), H), dtype=torch.uint8, device=DEV),
                         torch.zeros((int(cu[1]), H), dtype=torch.uint8, device=DEV),
                         torch.zeros((int(cu[1]), Hp), dtype=torch.uint8, device=DEV))
    rt.reset()
    # chunked after a reset: two updates give the one-shot result
    lengths = np.diff(z["c1_cu"])
    half = lengths // 2
    starts = z["c1_cu"][:-1]
    parts_out, parts_end = [], []
    for lo, hi in ((np.zeros_like(half), half), (half, lengths)):
        idx = np.concatenate([np.arange(s + a, s + b) for s, a, b in zip(starts, lo, hi)])
        ccu = torch.from_numpy(np.concatenate([[0], np.cumsum(hi - lo)]).astype(np.int32))
        o, e = rt.update_packed(ccu, torch.from_numpy(z["c1_q"][idx]).to(DEV),
                                torch.from_numpy(z["c1_k"][idx]).to(DEV),
                                torch.from_numpy(z["c1_payload"][idx]).to(DEV))
        parts_out.append((idx, o.cpu().numpy(), e.cpu().numpy()))
    got_out = np.empty_like(z["c1_out"])
    got_end = np.empty_like(z["c1_end"])
    for idx, o, e in parts_out:
        got_out[idx], got_end[idx] = o, e
    assert np.array_equal(got_out, z["c1_out"]) and np.array_equal(got_end, z["c1_end"])
    rt.close()
    with pytest.raises(RuntimeError, match="closed"):
        rt.reset()
