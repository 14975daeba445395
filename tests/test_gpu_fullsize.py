"""Parity at the benchmark configurations' full sizes.

The float64 oracle is quadratic-times-horizon, so at these sizes it checks sampled
(batch, head) slices; whole tensors are covered by size-independent properties of the
operator: linearity of the VJP in grad_output, agreement of the tensor-core and CUDA-core
contractions, packed == per-sequence dense, shard == unsharded, bit-exact hard outputs
against the (quadratic, exact) oracle matcher, and self-consistency of matched positions."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.helpers import grad_tol, nonzero_randn, normalised_error, repeated_stream_logits

DEV = "cuda"
GRAD_TOL = 1e-4


@pytest.fixture(scope="module")
def cabi():
    from rosa_soft_b200 import cabi as module
    module.load()
    return module


def _vjp(cabi, q, k, v, go, desc, W, scale, p, m, seed, mask=7, **kw):
    out, pq, pk, routes, _ = cabi.hard_forward(q, k, v, desc, W)
    seed_t = torch.tensor(seed, dtype=torch.int64, device=DEV) if p > 0 else None
    dq, dk, dv, _ = cabi.surrogate_vjp(q, k, v, go, desc, pq, pk, W, scale, p, m, seed_t, mask, **kw)
    return out, routes, dq, dk, dv


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_training_shape_sampled_slices_against_oracle(cabi, dtype):
    """README training shape: B=2 T=1024 H=64 D=8 Hv=16 Dv=8 W=128 p=0.1 m=3."""
    from oracle import rosa_oracle as orc
    B, T, H, D, Hv, Dv, W, p, m, seed = 2, 1024, 64, 8, 16, 8, 128, 0.1, 3.0, 2024
    group = H // Hv
    g = torch.Generator().manual_seed(1002)
    q, k = (torch.randn(B * T, H, D, generator=g).to(dtype).to(DEV) for _ in range(2))
    v = torch.randn(B * T, Hv, Dv, generator=g).to(dtype).to(DEV)
    go = torch.randn(B * T, H, Dv, generator=g).to(dtype).to(DEV)
    out, routes, dq, dk, dv = _vjp(cabi, q, k, v, go, (B, T), W, 1.0, p, m, seed)
    f = lambda t: t.float().cpu().numpy()
    cu = np.array([0, T], dtype=np.int64)
    for b, vh in ((0, 0), (1, 9), (1, 15)):       # one whole value-head group per sample
        rows, hs = slice(b * T, (b + 1) * T), slice(vh * group, (vh + 1) * group)
        ref_out, _ = orc.hard_forward(f(q[rows, hs]), f(k[rows, hs]), f(v[rows, vh:vh + 1]), cu, W)
        assert np.array_equal(f(out[rows, hs]), ref_out)
        rq, rk, rv = orc.surrogate_vjp(f(q[rows, hs]), f(k[rows, hs]), f(v[rows, vh:vh + 1]),
                                       f(go[rows, hs]), cu, W, 1.0, p, m, seed, batch_offset=b,
                                       head_offset=vh * group)
        assert normalised_error(f(dq[rows, hs]), rq) <= grad_tol(dtype)
        assert normalised_error(f(dk[rows, hs]), rk) <= grad_tol(dtype)
        assert normalised_error(f(dv[rows, vh:vh + 1]), rv) <= grad_tol(dtype)


def test_long_match_stress_full_length_properties(cabi):
    """Long-match stress at T=8192, D=2, Dv=16, W=256 (one batch element, 8 heads of the 64)."""
    from oracle import rosa_oracle as orc
    T, H, D, Hv, Dv, W = 8192, 8, 2, 8, 16, 256
    q = repeated_stream_logits(T, H, D, seed=1003, repeat_prob=0.3, seg=(16, 256)).to(torch.bfloat16).to(DEV)
    k = q.clone()
    v = nonzero_randn((T, Hv, Dv), 7, torch.bfloat16).to(DEV)
    g1 = nonzero_randn((T, H, Dv), 8, torch.bfloat16).to(DEV)
    g2 = nonzero_randn((T, H, Dv), 9, torch.bfloat16).to(DEV)
    out, routes, dq1, dk1, dv1 = _vjp(cabi, q, k, v, g1, (1, T), W, 1.0, 0.0, 3.0, 0)
    # hard output and routes: bit-exact against the exact quadratic matcher at full length
    f = lambda t: t.float().cpu().numpy()
    ref_out, ref_route = orc.hard_forward(f(q), f(k), f(v), np.array([0, T]), W)
    assert np.array_equal(f(out), ref_out)
    assert np.array_equal(routes.cpu().numpy(), np.where(ref_route > 0, ref_route, -1))
    assert (ref_route > 0).mean() > 0.9 and ref_route.max() > 0
    # the VJP is linear in grad_output (no dropout): vjp(g1 + g2) == vjp(g1) + vjp(g2)
    _, _, dq2, dk2, dv2 = _vjp(cabi, q, k, v, g2, (1, T), W, 1.0, 0.0, 3.0, 0)
    gsum = (g1.float() + g2.float())
    _, _, dqs, dks, dvs = _vjp(cabi, q.float(), k.float(), v.float(), gsum, (1, T), W, 1.0, 0.0, 3.0, 0)
    # (float32 rounding only: each row's logit adjoints sum to zero, so the long sums of this
    # stress case cancel and amplify the rounding noise to a few 1e-5 of the largest entry)
    for a, b, c in ((dq1, dq2, dqs), (dk1, dk2, dks), (dv1, dv2, dvs)):
        err = normalised_error((a + b).cpu().numpy(), c.cpu().numpy())
        assert err <= grad_tol(torch.bfloat16), err   # bf16-input runs against a float32-input run
    # tensor-core and CUDA-core contractions of the same tiles agree
    cc = _vjp(cabi, q, k, v, g1, (1, T), W, 1.0, 0.0, 3.0, 0, mask=7 | 0x100)[2:]
    for a, b in zip((dq1, dk1, dv1), cc):
        err = normalised_error(a.cpu().numpy(), b.cpu().numpy())
        assert err <= grad_tol(torch.bfloat16), err
    # the last key position of the sequence receives no gradient
    assert torch.all(dk1[T - 1] == 0) and torch.all(dv1[0] == 0)


def test_metric_shape_properties(cabi):
    """T=8192, D=8, Dv=8, W=128, dropout 0.1 (4 of the 64 heads): forward exact against the
    oracle matcher, sharded == unsharded, reproducible."""
    from oracle import rosa_oracle as orc
    T, H, D, Hv, Dv, W, p = 8192, 4, 8, 1, 8, 128, 0.1
    g = torch.Generator().manual_seed(5)
    q, k = (torch.randn(T, H, D, generator=g).bfloat16().to(DEV) for _ in range(2))
    v = torch.randn(T, Hv, Dv, generator=g).bfloat16().to(DEV)
    go = torch.randn(T, H, Dv, generator=g).bfloat16().to(DEV)
    out, routes, dq, dk, dv = _vjp(cabi, q, k, v, go, (1, T), W, 1.0, p, 3.0, 77,
                                   batch_offset=3, head_offset=8)
    f = lambda t: t.float().cpu().numpy()
    ref_out, _ = orc.hard_forward(f(q), f(k), f(v), np.array([0, T]), W)
    assert np.array_equal(f(out), ref_out)
    again = _vjp(cabi, q, k, v, go, (1, T), W, 1.0, p, 3.0, 77, batch_offset=3, head_offset=8)[2:]
    for a, b in zip((dq, dk, dv), again):
        assert torch.equal(a, b)
    # two-head shards with their global head offsets reproduce dQ/dK of the four-head run
    for h0 in (0, 2):
        sl = slice(h0, h0 + 2)
        _, _, sq, sk, _ = _vjp(cabi, q[:, sl].contiguous(), k[:, sl].contiguous(), v,
                               go[:, sl].contiguous(), (1, T), W, 1.0, p, 3.0, 77, batch_offset=3,
                               head_offset=8 + h0)
        assert torch.equal(sq, dq[:, sl]) and torch.equal(sk, dk[:, sl])


def test_packed_full_size_equals_per_sequence_dense(cabi):
    """32768 packed tokens, lengths uniform in [64, 4096], H=32 D=16 Hv=8 Dv=32 fp16 W=64 p=0.05 m=9
    (4 of the 32 heads): every sampled sequence equals a dense run with its ordinal as batch."""
    rng = np.random.default_rng(1004)
    lengths, total = [], 0
    while total < 32768:
        n = min(int(rng.integers(64, 4097)), 32768 - total)
        lengths.append(n)
        total += n
    N, H, D, Hv, Dv, W, p, m, seed = 32768, 4, 16, 1, 32, 64, 0.05, 9.0, 31337
    cu_np = np.concatenate([[0], np.cumsum(lengths)])
    g = torch.Generator().manual_seed(1004)
    q, k = (torch.randn(N, H, D, generator=g).half().to(DEV) for _ in range(2))
    v = torch.randn(N, Hv, Dv, generator=g).half().to(DEV)
    go = torch.randn(N, H, Dv, generator=g).half().to(DEV)
    cu = torch.from_numpy(cu_np.astype(np.int32)).to(DEV)
    out, routes, dq, dk, dv = _vjp(cabi, q, k, v, go, cu, W, 1.0, p, m, seed)
    order = np.argsort(lengths)
    for s in (int(order[0]), int(order[len(order) // 2]), int(order[-1])):
        a, b = int(cu_np[s]), int(cu_np[s + 1])
        rows = slice(a, b)
        o2, r2, q2, k2, v2 = _vjp(cabi, q[rows].contiguous(), k[rows].contiguous(),
                                  v[rows].contiguous(), go[rows].contiguous(), (1, b - a), W, 1.0,
                                  p, m, seed, batch_offset=s)
        assert torch.equal(o2, out[rows])
        assert torch.equal(torch.where(r2 >= 0, r2 + a, r2), routes[rows])
        assert torch.equal(q2, dq[rows]) and torch.equal(k2, dk[rows]) and torch.equal(v2, dv[rows])


def test_hard_inference_full_length_streams(cabi):
    """T=16384 streams of 32-bit symbols with planted copies: sampled streams bit-exact against
    the oracle, and every reported match of the whole batch is a real, causal match."""
    import importlib.util, os
    from oracle import rosa_oracle as orc
    spec = importlib.util.spec_from_file_location(
        "bench_inputs", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    cfg = dict(B=8, T=16384, H=8, Hv=8, Dv=8)
    qs, ks, pay = bench.make_inference_inputs(cfg, 1005, DEV)
    B, T, H = cfg["B"], cfg["T"], cfg["H"]
    W = 32
    out, end, _ = cabi.hard_inference(qs.reshape(B * T, H), ks.reshape(B * T, H),
                                      pay.reshape(B * T, 8, 8), (B, T), W)
    end = end.reshape(B, T, H)
    out = out.reshape(B, T, H, 8)
    for b in (0, 5):
        ro, re = orc.hard_inference(qs[b].cpu().numpy().view(np.uint32), ks[b].cpu().numpy().view(np.uint32),
                                    pay[b].cpu().numpy(), np.array([0, T]), W)
        assert np.array_equal(end[b].cpu().numpy(), re)
        assert np.array_equal(out[b].cpu().numpy(), ro)
    hit = end >= 0
    assert 0.2 < hit.float().mean().item() < 1.0
    pos = torch.arange(T, device=DEV).view(1, T, 1)
    assert torch.all(end[hit] < pos.expand_as(end)[hit])                 # strictly causal
    idx = end.clamp_min(0)
    assert torch.all(torch.gather(ks, 1, idx)[hit] == qs[hit])           # last symbol matches
    succ = torch.gather(pay, 1, (idx + 1).clamp_max(T - 1).unsqueeze(-1).expand(B, T, H, 8))
    assert torch.equal(succ[hit], out[hit]) and not out[~hit].any()      # successor payload
