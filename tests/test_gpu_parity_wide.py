"""GPU parity, second part: every kernel instantiation that the benchmark configurations use
meets the float64 oracle directly.

* value rows of 9..32 components (the 4- and 8-group utility tables and the 16/32-column
  tensor-core operands) crossed with narrow and wide symbols, with and without dropout and a
  closing horizon window;
* the long-match stress configuration at its full length (T = 8192, D = 2, Dv = 16, W = 256:
  matches sit on the horizon for hundreds of rows, the cancellation regime of the windowed
  adjoint) on whole (batch, head) slices;
* the packed configuration (32768 tokens, D = 16, Dv = 32, fp16, dropout) on its shortest, a
  median and its longest sequence, the sequence ordinal as the dropout batch coordinate;
* the fall-back matchers: rows with more genuine candidates than the hashed prefilter accepts
  (run-length matcher re-launch and atomicMax merge), and horizons of 2048 and more (64-bit
  candidate keys);
* packed symbols word for word, signed zeros / NaN / infinities included;
* element-wise closeness (rtol / atol) beside the normalised maximum error.
"""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import rosa_oracle as orc
from tests.helpers import (TORCH_DTYPES, assert_grads_close, grad_tol, nonzero_randn, normalised_error,
                           oracle_forward, oracle_grads, repeated_stream_logits)

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda"
GRAD_TOL = 1e-4


@pytest.fixture(scope="module")
def cabi():
    from rosa_soft_b200 import cabi as module
    module.load()
    return module


def _run(cabi, q, k, v, go, desc, W, scale, p, m, seed, mask=7, **kw):
    out, pq, pk, routes, _ = cabi.hard_forward(q, k, v, desc, W)
    seed_t = torch.tensor(seed, dtype=torch.int64, device=DEV) if p > 0 else None
    dq, dk, dv, ws = cabi.surrogate_vjp(q, k, v, go, desc, pq, pk, W, scale, p, m, seed_t, mask, **kw)
    torch.cuda.synchronize()
    assert cabi.read_status(ws) == 0
    return out, pq, pk, routes, dq, dk, dv


# T, H, D, Hv, Dv, W, scale, p, m, dtype: three VJP bands each, so the band / item bookkeeping
# of every instantiation is walked as well
WIDE_SHAPES = [
    (600, 2, 2, 2, 12, 30, 1.0, 0.0, 3.0, torch.float32),
    (600, 2, 2, 1, 16, 700, 1.0, 0.1, 3.0, torch.bfloat16),     # horizon never closes
    (530, 2, 2, 2, 24, 64, 0.7, 0.0, 3.0, torch.float32),
    (530, 2, 2, 2, 32, 16, 1.0, 0.2, 2.0, torch.float16),
    (560, 2, 16, 1, 12, 64, 1.0, 0.05, 9.0, torch.float16),
    (560, 2, 16, 2, 16, 40, 1.3, 0.0, 3.0, torch.float32),
    (560, 4, 16, 1, 24, 600, 1.0, 0.1, 3.0, torch.float32),
    (600, 4, 16, 1, 32, 64, 1.0, 0.05, 9.0, torch.float16),     # the packed benchmark's controls
    (520, 2, 20, 2, 12, 9, 1.0, 0.0, 3.0, torch.bfloat16),
    (520, 2, 20, 1, 16, 128, 1.0, 0.3, 3.0, torch.float32),
    (520, 2, 20, 2, 24, 520, 2.0, 0.0, 1.5, torch.float32),
    (520, 2, 20, 1, 32, 33, 1.0, 0.1, 3.0, torch.float32),
    (300, 2, 8, 1, 16, 20, 11.0, 0.1, 3.0, torch.float32),      # per-row softmax maximum path
    (300, 2, 3, 1, 32, 20, 10.0, 0.0, 3.0, torch.float32),
]


@pytest.mark.parametrize("shape", WIDE_SHAPES)
def test_value_widths_and_symbol_widths_against_oracle(cabi, shape):
    T, H, D, Hv, Dv, W, scale, p, m, dt = shape
    seed = 3000 + 7 * D + Dv
    if D <= 2:   # narrow symbols: a repeated stream, so matches are long and the window closes
        q = repeated_stream_logits(T, H, D, seed=seed).to(dt).to(DEV)
        k = q.clone()
    else:
        q = nonzero_randn((T, H, D), seed, dt).to(DEV)
        k = nonzero_randn((T, H, D), seed + 1, dt).to(DEV)
    v = nonzero_randn((T, Hv, Dv), seed + 2, dt).to(DEV)
    go = nonzero_randn((T, H, Dv), seed + 3, dt).to(DEV)
    cu = np.array([0, T], dtype=np.int64)
    out, pq, pk, routes, dq, dk, dv = _run(cabi, q, k, v, go, (1, T), W, scale, p, m, 99)
    ref_out, ref_route = oracle_forward(q, k, v, cu, W)
    assert np.array_equal(out.float().cpu().numpy(), ref_out)
    assert np.array_equal(routes.cpu().numpy(), np.where(ref_route > 0, ref_route, -1))
    rq, rk, rv = oracle_grads(q, k, v, go, cu, W, scale, p, m, 99)
    for name, mine, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        err = normalised_error(mine.cpu().numpy(), ref)
        assert err <= grad_tol(dt), (name, err)
    # both contraction paths of the second sweep meet the oracle, not only each other
    cc = _run(cabi, q, k, v, go, (1, T), W, scale, p, m, 99, mask=7 | 0x100)[4:]
    for name, mine, ref in (("dq", cc[0], rq), ("dk", cc[1], rk), ("dv", cc[2], rv)):
        err = normalised_error(mine.cpu().numpy(), ref)
        assert err <= GRAD_TOL, (name + " (CUDA-core contraction)", err)


def test_long_match_stress_full_length_against_oracle(cabi):
    """T = 8192, D = 2, Dv = 16, W = 256, bf16: whole (batch, head) slices against the float64
    oracle.  Head 0 is the benchmark's stream (repeated segments of 16..256 tokens: matches of up
    to 255 symbols); head 1 repeats segments of up to 700 tokens, so matches sit on the horizon for
    hundreds of rows and the window products of the adjoint stay alive (the cancellation regime)."""
    T, H, D, Hv, Dv, W = 8192, 2, 2, 2, 16, 256
    q = torch.cat([repeated_stream_logits(T, 1, D, seed=1003, repeat_prob=0.3, seg=(16, 256)),
                   repeated_stream_logits(T, 1, D, seed=1004, repeat_prob=0.4, seg=(16, 700))], dim=1)
    q = q.to(torch.bfloat16).to(DEV)
    k = q.clone()
    v = nonzero_randn((T, Hv, Dv), 7, torch.bfloat16).to(DEV)
    go = nonzero_randn((T, H, Dv), 8, torch.bfloat16).to(DEV)
    cu = np.array([0, T], dtype=np.int64)
    out, pq, pk, routes, dq, dk, dv = _run(cabi, q, k, v, go, (1, T), W, 1.0, 0.0, 3.0, 0)
    ref_out, ref_route = oracle_forward(q, k, v, cu, W)
    assert np.array_equal(out.float().cpu().numpy(), ref_out)
    assert np.array_equal(routes.cpu().numpy(), np.where(ref_route > 0, ref_route, -1))
    _, ref_len = orc.hard_routes(orc.pack_symbols(q.float().cpu().numpy()),
                                 orc.pack_symbols(k.float().cpu().numpy()), cu, W)
    assert (ref_len[:, 0] >= 128).mean() > 0.05   # long matches in the benchmark's stream
    assert (ref_len[:, 1] == W).mean() > 0.05     # and matches that sit on the horizon
    rq, rk, rv = oracle_grads(q, k, v, go, cu, W, 1.0, 0.0, 3.0, 0)
    for name, mine, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        for h in range(H):
            hv = slice(h, h + 1)
            err = normalised_error(mine[:, hv].cpu().numpy(), ref[:, hv])
            assert err <= grad_tol(torch.bfloat16), (name, h, err)


def test_packed_configuration_sequences_against_oracle(cabi):
    """32768 packed tokens, lengths uniform in [64, 4096], D = 16, Dv = 32, fp16, W = 64, p = 0.05,
    m = 9 (one value-head group of 4 heads): the shortest, a median and the longest sequence of
    the packed run against the oracle with the sequence ordinal as batch coordinate."""
    rng = np.random.default_rng(1004)
    lengths, total = [], 0
    while total < 32768:
        n = min(int(rng.integers(64, 4097)), 32768 - total)
        lengths.append(n)
        total += n
    assert max(lengths) >= 2048
    N, H, D, Hv, Dv, W, p, m, seed = 32768, 4, 16, 1, 32, 64, 0.05, 9.0, 31337
    cu_np = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)
    g = torch.Generator().manual_seed(1004)
    q, k = (torch.randn(N, H, D, generator=g).half().to(DEV) for _ in range(2))
    v = torch.randn(N, Hv, Dv, generator=g).half().to(DEV)
    go = torch.randn(N, H, Dv, generator=g).half().to(DEV)
    cu = torch.from_numpy(cu_np.astype(np.int32)).to(DEV)
    out, pq, pk, routes, dq, dk, dv = _run(cabi, q, k, v, go, cu, W, 1.0, p, m, seed)
    f = lambda t: t.float().cpu().numpy()
    order = np.argsort(lengths)
    for s in (int(order[0]), int(order[len(order) // 2]), int(order[-1])):
        a, b = int(cu_np[s]), int(cu_np[s + 1])
        rows = slice(a, b)
        one = np.array([0, b - a], dtype=np.int64)
        ref_out, ref_route = orc.hard_forward(f(q[rows]), f(k[rows]), f(v[rows]), one, W)
        assert np.array_equal(f(out[rows]), ref_out)
        assert np.array_equal(routes[rows].cpu().numpy(), np.where(ref_route > 0, ref_route + a, -1))
        rq, rk, rv = orc.surrogate_vjp(f(q[rows]), f(k[rows]), f(v[rows]), f(go[rows]), one, W, 1.0,
                                       p, m, seed, batch_offset=s)
        for name, mine, ref in (("dq", dq[rows], rq), ("dk", dk[rows], rk), ("dv", dv[rows], rv)):
            err = normalised_error(f(mine), ref)
            assert err <= grad_tol(torch.float16), (s, name, err)
        # after the cast to the input dtype the reference's own fp16 tolerance holds as well
        assert normalised_error(f(dv[rows].half()), rv) <= 3e-3


# ------------------------------------------------------------------ fall-back matchers

def _two_symbol_stream(T, H, bits, seed):
    """Random stream over two symbols of `bits` bits: about half of the earlier positions agree
    with a row's last symbol (genuine candidates by the thousand), yet matches stay a dozen
    symbols long, so no row ever stops early on a match at the horizon."""
    rng = np.random.default_rng(seed)
    pair = rng.integers(1 << (bits - 1), 1 << bits, size=(2, H), dtype=np.uint64).astype(np.uint32)
    pick = rng.integers(0, 2, size=(T, H))
    return np.where(pick == 1, pair[1][None, :], pair[0][None, :]).astype(np.uint32)


def test_wide_symbol_rows_beyond_the_prefilter_limit_take_the_run_length_matcher(cabi):
    """Streams of 32-bit symbols over a two-symbol alphabet give every late row thousands of
    genuine candidates: the hashed prefilter raises its flag, the run-length matcher redoes the
    launch and merges into the rows the prefilter had already resolved (a random wide-symbol head
    and a short sequence stay with the prefilter)."""
    T, H, Hp, Dp, W = 6200, 3, 1, 2, 50
    k = _two_symbol_stream(T, H, 32, 5)
    rng = np.random.default_rng(6)
    k[:, 2] = rng.integers(0, 1 << 32, size=T, dtype=np.uint64).astype(np.uint32)   # a random head
    # the query stream is drawn independently over the same two symbols (a shifted copy of the
    # keys would match at the horizon on every row and stop the prefilter at once)
    pick = rng.integers(0, 2, size=(T, H))
    q = np.where(pick == 1, k.max(axis=0)[None, :], k.min(axis=0)[None, :]).astype(np.uint32)
    q[:, 2] = k[:, 2]
    pay = rng.standard_normal((T, Hp, Dp)).astype(np.float32)
    cu_np = np.array([0, 300, 300, T], dtype=np.int64)
    ref_out, ref_end = orc.hard_inference(q, k, pay, cu_np, W)
    out, end, ws = cabi.hard_inference(torch.from_numpy(q.view(np.int32)).to(DEV),
                                       torch.from_numpy(k.view(np.int32)).to(DEV),
                                       torch.from_numpy(pay).to(DEV),
                                       torch.from_numpy(cu_np.astype(np.int32)).to(DEV), W)
    assert np.array_equal(end.cpu().numpy(), ref_end)
    assert np.array_equal(out.cpu().numpy(), ref_out)
    assert cabi.read_status(ws) == 0
    # the flag word of the plan says that the fall-back really ran
    assert ws[:16].view(torch.int32).cpu().numpy()[2] == 1


def test_training_forward_with_wide_two_symbol_stream(cabi):
    """The training forward with D = 12 (hashed prefilter) on a two-symbol stream: same
    fall-back, checked through the operator's outputs."""
    T, H, D, Hv, Dv, W = 6200, 2, 12, 1, 4, 64
    sym = _two_symbol_stream(T, H, D, 9)
    bits = (sym[..., None] >> np.arange(D)) & 1
    q = torch.from_numpy(np.where(bits, 0.6, -0.6).astype(np.float32)).to(DEV)
    k = q.clone()
    v = nonzero_randn((T, Hv, Dv), 3).to(DEV)
    out, pq, pk, routes, ws = cabi.hard_forward(q, k, v, (1, T), W)
    ref_out, ref_route = oracle_forward(q, k, v, np.array([0, T]), W)
    assert np.array_equal(out.cpu().numpy(), ref_out)
    assert np.array_equal(routes.cpu().numpy(), np.where(ref_route > 0, ref_route, -1))
    assert ws[:16].view(torch.int32).cpu().numpy()[2] == 1


def test_horizon_beyond_the_narrow_key_range_takes_the_generic_matcher(cabi):
    """W >= 2048: a constant stretch of 3000 symbols (matches up to the horizon of 2500) followed
    by a two-symbol stream whose rows overflow the prefilter: the generic run-length matcher
    (64-bit candidate keys) redoes the launch."""
    T, H, W = 7400, 2, 2500
    k = _two_symbol_stream(T, H, 32, 4)
    k[:3000] = k[0]                            # constant start: one of the two symbols per head
    q = _two_symbol_stream(T, H, 32, 4)        # same alphabet (same seed), then reshuffled
    q = q[np.random.default_rng(11).permutation(T)]
    q[:3000] = k[:3000]
    pay = np.random.default_rng(8).standard_normal((T, 1, 2)).astype(np.float32)
    cu_np = np.array([0, T], dtype=np.int64)
    ref_out, ref_end = orc.hard_inference(q, k, pay, cu_np, W)
    out, end, ws = cabi.hard_inference(torch.from_numpy(q.view(np.int32)).to(DEV),
                                       torch.from_numpy(k.view(np.int32)).to(DEV),
                                       torch.from_numpy(pay).to(DEV), (1, T), W)
    assert np.array_equal(end.cpu().numpy(), ref_end)
    assert np.array_equal(out.cpu().numpy(), ref_out)
    assert ws[:16].view(torch.int32).cpu().numpy()[2] == 1
    _, ref_len = orc.hard_routes(q, k, cu_np, W)
    assert ref_len.max() == W


# ------------------------------------------------------------------ packed symbols

@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [1, 2, 8, 13, 32])
def test_packed_symbols_equal_the_oracle_word_for_word(cabi, D, dt):
    B, T, H = 3, 70, 5
    q = nonzero_randn((B * T, H, D), 40 + D, dt)
    k = nonzero_randn((B * T, H, D), 41 + D, dt)
    # signed zeros, NaN and infinities: only strictly positive components set their bit
    specials = torch.tensor([0.0, -0.0, float("nan"), float("inf"), -float("inf")]).to(dt)
    flat_q, flat_k = q.view(-1), k.view(-1)
    flat_q[::7] = specials.repeat(flat_q[::7].numel() // 5 + 1)[:flat_q[::7].numel()]
    flat_k[3::11] = specials.repeat(flat_k[3::11].numel() // 5 + 1)[:flat_k[3::11].numel()]
    v = nonzero_randn((B * T, 1, 3), 42, dt)
    want_q = orc.pack_symbols(q.float().numpy()).astype(np.int64).view(np.int64)
    want_k = orc.pack_symbols(k.float().numpy()).astype(np.int64)
    as_u32 = lambda t: t.cpu().numpy().view(np.uint32).astype(np.int64)
    # dense layout [B, H, T]
    _, pq, pk, _, _ = cabi.hard_forward(q.to(DEV), k.to(DEV), v.to(DEV), (B, T), 8)
    assert pq.shape == (B, H, T) and pq.dtype == torch.int32 and pq.is_contiguous()
    assert np.array_equal(as_u32(pq).transpose(0, 2, 1).reshape(B * T, H), want_q)
    assert np.array_equal(as_u32(pk).transpose(0, 2, 1).reshape(B * T, H), want_k)
    # packed layout [H, N]
    cu = torch.tensor([0, 1, 1, 100, B * T], dtype=torch.int32, device=DEV)
    _, pq, pk, _, _ = cabi.hard_forward(q.to(DEV), k.to(DEV), v.to(DEV), cu, 8)
    assert pq.shape == (H, B * T) and pq.is_contiguous()
    assert np.array_equal(as_u32(pq).T, want_q) and np.array_equal(as_u32(pk).T, want_k)


def test_nonfinite_inputs_follow_the_reference_policy(cabi):
    """Fixture produced by the reference (its policy test, tests/test_soft_cuda.py:570-611, with
    signed zeros added): NaN gradients appear exactly where the reference has them, the rest
    agrees, the never-used last key row is an exact zero."""
    z = np.load(os.path.join(GOLDEN, "nonfinite_f32_policy.npz"))
    B, T = z["q"].shape[:2]
    flat = lambda a: torch.from_numpy(a).reshape((B * T,) + a.shape[2:]).to(DEV)
    q, k, v, go = flat(z["q"]), flat(z["k"]), flat(z["v"]), flat(z["go"])
    out, pq, pk, routes, dq, dk, dv = _run(cabi, q, k, v, go, (B, T), int(z["W"]), float(z["scale"]),
                                           0.0, float(z["m"]), 0)
    assert np.array_equal(out.cpu().numpy().reshape(z["out"].shape), z["out"])
    assert np.array_equal(pq.cpu().numpy().reshape(-1).view(np.uint32),
                          orc.pack_symbols(z["q"].reshape(B * T, 1, -1)).reshape(-1))
    for name, mine in (("dq", dq), ("dk", dk), ("dv", dv)):
        ref = z[name].reshape(mine.shape)
        got = mine.cpu().numpy()
        assert np.array_equal(np.isnan(got), np.isnan(ref)), name
        ok = np.isfinite(ref)
        assert np.allclose(got[ok], ref[ok], rtol=2e-5, atol=2e-6), name
    assert torch.all(dk[T - 1] == 0)


# ------------------------------------------------------------------ element-wise closeness

def _fixture_names():
    import glob
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "dense_*.npz")))


@pytest.mark.parametrize("name", _fixture_names())
def test_fixture_gradients_are_close_element_by_element(cabi, name):
    """The reference's own fixtures under an allclose-style bound: |mine - ref| <= rtol |ref| + atol
    with atol a small fraction of the tensor's largest entry (1e-4 / 2e-5 for float32 and float64
    inputs; the reference's 2e-2 and 3e-3 after the cast for bfloat16 and float16)."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    dt = TORCH_DTYPES[str(z["dtype"])]
    B, T = z["q"].shape[:2]
    flat = lambda a: torch.from_numpy(a.astype(np.float32)).reshape((B * T,) + a.shape[2:]).to(DEV, dt)
    q, k, v, go = flat(z["q"]), flat(z["k"]), flat(z["v"]), flat(z["go"])
    _, _, _, _, dq, dk, dv = _run(cabi, q, k, v, go, (B, T), int(z["W"]), float(z["scale"]),
                                  float(z["p"]), float(z["m"]), int(z["dropout_seed"]))
    for label, mine, ref in (("dq", dq, z["dq"]), ("dk", dk, z["dk"]), ("dv", dv, z["dv"])):
        assert_grads_close(mine, ref, str(z["dtype"]), name + ":" + label)
