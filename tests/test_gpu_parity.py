"""GPU parity: the CUDA path (through the C ABI and through torch.ops) against the CPU
oracle and the committed reference fixtures.  Hard outputs, packed symbols and routes are
bit-exact; gradients are compared in float32 (the operator's own output type) against the
float64 oracle with a normalised max error of 1e-4, and after the cast to the input dtype
with the reference's own half-precision tolerances."""
import glob
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests.helpers import (TORCH_DTYPES, grad_tol, nonzero_randn, normalised_error, oracle_forward,
                           oracle_grads, repeated_stream_logits)

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
GRAD_TOL = 1e-4   # float32 gradients vs the float64 oracle, normalised by the tensor max
CAST_TOL = {"float64": 1e-4, "float32": 1e-4, "bfloat16": 2e-2, "float16": 3e-3}
DEV = "cuda"


@pytest.fixture(scope="module")
def cabi():
    from rosa_soft_b200 import cabi as module
    module.load()
    return module


@pytest.fixture(scope="module")
def ops():
    import rosa_soft_b200
    return rosa_soft_b200


def _fixture_names(kind):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, kind + "_*.npz")))


def _run_cabi(cabi, q, k, v, go, cu_desc, W, scale, p, m, seed, mask=7):
    out, pq, pk, routes, ws = cabi.hard_forward(q, k, v, cu_desc, W)
    seed_t = torch.tensor(seed, dtype=torch.int64, device=DEV) if p > 0 else None
    dq, dk, dv, ws2 = cabi.surrogate_vjp(q, k, v, go, cu_desc, pq, pk, W, scale, p, m, seed_t, mask)
    torch.cuda.synchronize()
    return out, pq, pk, routes, dq, dk, dv


@pytest.mark.parametrize("name", _fixture_names("dense"))
def test_dense_fixture_through_c_abi(cabi, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    dt = TORCH_DTYPES[str(z["dtype"])]
    B, T, H, D = z["q"].shape
    flat = lambda a: torch.from_numpy(a.astype(np.float32)).reshape((B * T,) + a.shape[2:]).to(DEV, dt)
    q, k, v, go = flat(z["q"]), flat(z["k"]), flat(z["v"]), flat(z["go"])
    out, pq, pk, routes, dq, dk, dv = _run_cabi(cabi, q, k, v, go, (B, T), int(z["W"]),
                                                float(z["scale"]), float(z["p"]), float(z["m"]),
                                                int(z["dropout_seed"]))
    assert np.array_equal(out.float().cpu().numpy().reshape(z["out"].shape),
                          z["out"].astype(np.float32))
    local = routes.cpu().numpy().reshape(B, T, H)
    local = np.where(local < 0, 0, local - (np.arange(B) * T)[:, None, None])
    assert np.array_equal(local.transpose(0, 2, 1), z["routes"])
    tol = CAST_TOL[str(z["dtype"])]
    for mine, ref in ((dq, z["dq"]), (dk, z["dk"]), (dv, z["dv"])):
        assert normalised_error(mine.cpu().numpy(), ref) <= tol


@pytest.mark.parametrize("name", _fixture_names("varlen"))
def test_varlen_fixture_through_c_abi(cabi, name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    dt = TORCH_DTYPES[str(z["dtype"])]
    dev = lambda a: torch.from_numpy(a.astype(np.float32)).to(DEV, dt)
    q, k, v, go = dev(z["q"]), dev(z["k"]), dev(z["v"]), dev(z["go"])
    cu = torch.from_numpy(z["cu_seqlens"]).to(DEV)
    out, pq, pk, routes, dq, dk, dv = _run_cabi(cabi, q, k, v, go, cu, int(z["W"]),
                                                float(z["scale"]), float(z["p"]), float(z["m"]),
                                                int(z["dropout_seed"]))
    assert np.array_equal(out.float().cpu().numpy(), z["out"].astype(np.float32))
    starts = np.repeat(z["cu_seqlens"][:-1], np.diff(z["cu_seqlens"]))
    local = routes.cpu().numpy()
    local = np.where(local < 0, 0, local - starts[:, None])
    assert np.array_equal(local, z["routes"])
    for mine, ref in ((dq, z["dq"]), (dk, z["dk"]), (dv, z["dv"])):
        assert normalised_error(mine.cpu().numpy(), ref) <= CAST_TOL[str(z["dtype"])]


SHAPES = [
    # B, T, H, D, Hv, Dv, W, scale, p, m, dtype
    (1, 33, 2, 16, 1, 5, 16, 1.0, 0.0, 3.0, torch.float32),
    (2, 300, 4, 3, 2, 8, 40, 1.3, 0.1, 2.0, torch.float32),      # two VJP bands
    (1, 700, 2, 8, 1, 8, 128, 1.0, 0.1, 3.0, torch.bfloat16),    # three bands, window closes
    (1, 1100, 1, 2, 1, 4, 700, 0.7, 0.0, 3.0, torch.float32),    # two forward work items
    (1, 137, 2, 32, 2, 3, 200, 1.0, 0.0, 3.0, torch.float16),    # D = 32, W > T
    (1, 64, 6, 5, 3, 40, 9, 1.0, 0.2, 9.0, torch.float32),       # grouped heads, Dv > 32
    (1, 20, 1, 4, 1, 3000, 4, 1.0, 0.0, 3.0, torch.float32),     # very wide value rows
    (3, 1, 2, 3, 1, 2, 4, 1.0, 0.0, 3.0, torch.float32),         # singleton sequences
    (2, 2, 1, 1, 1, 1, 1, 1.0, 0.0, 3.0, torch.float32),
    (1, 290, 2, 4, 1, 8, 200, 9.0, 0.1, 3.0, torch.float32),     # large scale: per-row softmax max
    (1, 150, 2, 6, 1, 36, 60, 12.0, 0.0, 2.0, torch.float32),    # same with wide value rows
]


@pytest.mark.parametrize("shape", SHAPES)
def test_random_dense_against_oracle(cabi, shape):
    B, T, H, D, Hv, Dv, W, scale, p, m, dt = shape
    seed = 1000 + T
    q = nonzero_randn((B * T, H, D), seed, dt).to(DEV)
    k = nonzero_randn((B * T, H, D), seed + 1, dt).to(DEV)
    v = nonzero_randn((B * T, Hv, Dv), seed + 2, dt).to(DEV)
    go = nonzero_randn((B * T, H, Dv), seed + 3, dt).to(DEV)
    cu = np.arange(B + 1, dtype=np.int64) * T
    out, pq, pk, routes, dq, dk, dv = _run_cabi(cabi, q, k, v, go, (B, T), W, scale, p, m, 77)
    ref_out, ref_route = oracle_forward(q, k, v, cu, W)
    assert np.array_equal(out.float().cpu().numpy(), ref_out)
    starts = np.repeat(cu[:-1], T)
    want = np.where(ref_route > 0, ref_route + starts[:, None], -1)
    assert np.array_equal(routes.cpu().numpy(), want)
    rq, rk, rv = oracle_grads(q, k, v, go, cu, W, scale, p, m, 77)
    for mine, ref in ((dq, rq), (dk, rk), (dv, rv)):
        assert normalised_error(mine.cpu().numpy(), ref) <= grad_tol(dt)


@pytest.mark.parametrize("bits,W,T", [(2, 16, 600), (1, 8, 300), (2, 300, 520)])
def test_long_match_stress_against_oracle(cabi, bits, W, T):
    """Repeated token segments: hard matches reach the horizon and the windowed adjoint
    (the ring of S-bar * P terms) is exercised."""
    H, Hv, Dv = 2, 2, 6
    q = repeated_stream_logits(T, H, bits, seed=5 + T).to(DEV)
    k = q.clone()
    v = nonzero_randn((T, Hv, Dv), 11).to(DEV)
    go = nonzero_randn((T, H, Dv), 12).to(DEV)
    cu = np.array([0, T], dtype=np.int64)
    out, pq, pk, routes, dq, dk, dv = _run_cabi(cabi, q, k, v, go, (1, T), W, 1.0, 0.0, 3.0, 0)
    ref_out, ref_route = oracle_forward(q, k, v, cu, W)
    assert np.array_equal(out.float().cpu().numpy(), ref_out)
    assert np.array_equal(routes.cpu().numpy(), np.where(ref_route > 0, ref_route, -1))
    rq, rk, rv = oracle_grads(q, k, v, go, cu, W, 1.0, 0.0, 3.0, 0)
    for mine, ref in ((dq, rq), (dk, rk), (dv, rv)):
        assert normalised_error(mine.cpu().numpy(), ref) <= GRAD_TOL


def test_all_match_whole_sequence(cabi):
    """All-ones inputs: every diagonal is one exact run much longer than the horizon."""
    T, H, D, Dv, W = 900, 1, 4, 4, 12
    q = torch.ones(T, H, D, device=DEV)
    k = torch.ones(T, H, D, device=DEV)
    v = nonzero_randn((T, 1, Dv), 3).to(DEV)
    go = nonzero_randn((T, H, Dv), 4).to(DEV)
    cu = np.array([0, T], dtype=np.int64)
    out, pq, pk, routes, dq, dk, dv = _run_cabi(cabi, q, k, v, go, (1, T), W, 1.0, 0.0, 3.0, 0)
    ref_out, ref_route = oracle_forward(q, k, v, cu, W)
    assert np.array_equal(out.float().cpu().numpy(), ref_out)
    rq, rk, rv = oracle_grads(q, k, v, go, cu, W, 1.0, 0.0, 3.0, 0)
    for mine, ref in ((dq, rq), (dk, rk), (dv, rv)):
        assert normalised_error(mine.cpu().numpy(), ref) <= GRAD_TOL


@pytest.mark.parametrize("mask", range(1, 8))
def test_gradient_masks(cabi, mask):
    T, H, D, Hv, Dv, W = 90, 2, 4, 1, 5, 7
    q = nonzero_randn((T, H, D), 31).to(DEV)
    k = nonzero_randn((T, H, D), 32).to(DEV)
    v = nonzero_randn((T, Hv, Dv), 33).to(DEV)
    go = nonzero_randn((T, H, Dv), 34).to(DEV)
    full = _run_cabi(cabi, q, k, v, go, (1, T), W, 1.0, 0.1, 3.0, 9)[4:]
    part = _run_cabi(cabi, q, k, v, go, (1, T), W, 1.0, 0.1, 3.0, 9, mask=mask)[4:]
    for bit, (a, b) in enumerate(zip(part, full)):
        if mask >> bit & 1:
            assert torch.equal(a, b)
        else:
            assert a is None


def test_tensor_core_and_cuda_core_contractions_agree(cabi):
    """The tcgen05 contraction (bf16 high/low operand pairs, fp32 accumulation in tensor
    memory) against the plain CUDA-core contraction of the same tiles."""
    for dt, T, D, Dv, W, p in ((torch.float32, 700, 8, 8, 64, 0.1), (torch.bfloat16, 300, 16, 32, 40, 0.0),
                               (torch.float16, 290, 20, 12, 9, 0.0)):
        H, Hv = 2, 1
        q = nonzero_randn((T, H, D), 141, dt).to(DEV)
        k = nonzero_randn((T, H, D), 142, dt).to(DEV)
        v = nonzero_randn((T, Hv, Dv), 143, dt).to(DEV)
        go = nonzero_randn((T, H, Dv), 144, dt).to(DEV)
        tc = _run_cabi(cabi, q, k, v, go, (1, T), W, 1.0, p, 3.0, 5)[4:]
        cc = _run_cabi(cabi, q, k, v, go, (1, T), W, 1.0, p, 3.0, 5, mask=7 | 0x100)[4:]
        for x, y in zip(tc, cc):
            assert normalised_error(x.cpu().numpy(), y.cpu().numpy()) <= max(2e-5, grad_tol(dt) / 2)


def test_backward_is_bitwise_reproducible(cabi):
    T, H, D, Hv, Dv, W = 1500, 4, 3, 2, 8, 33
    q = repeated_stream_logits(T, H, D, seed=8).to(DEV)
    k = q.clone()
    v = nonzero_randn((T, Hv, Dv), 41).to(DEV)
    go = nonzero_randn((T, H, Dv), 42).to(DEV)
    a = _run_cabi(cabi, q, k, v, go, (1, T), W, 1.0, 0.1, 3.0, 5)[4:]
    b = _run_cabi(cabi, q, k, v, go, (1, T), W, 1.0, 0.1, 3.0, 5)[4:]
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_varlen_random_against_oracle_and_dense(cabi):
    lengths = [5, 0, 300, 1, 2, 259, 0, 64]
    N, H, D, Hv, Dv, W = sum(lengths), 4, 6, 2, 7, 50
    cu_np = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)
    q = nonzero_randn((N, H, D), 51).to(DEV)
    k = nonzero_randn((N, H, D), 52).to(DEV)
    v = nonzero_randn((N, Hv, Dv), 53).to(DEV)
    go = nonzero_randn((N, H, Dv), 54).to(DEV)
    cu = torch.from_numpy(cu_np.astype(np.int32)).to(DEV)
    out, pq, pk, routes, dq, dk, dv = _run_cabi(cabi, q, k, v, go, cu, W, 1.0, 0.15, 3.0, 1234567)
    ref_out, ref_route = oracle_forward(q, k, v, cu_np, W)
    assert np.array_equal(out.float().cpu().numpy(), ref_out)
    assert pq.shape == (H, N) and pq.dtype == torch.int32
    rq, rk, rv = oracle_grads(q, k, v, go, cu_np, W, 1.0, 0.15, 3.0, 1234567)
    for mine, ref in ((dq, rq), (dk, rk), (dv, rv)):
        assert normalised_error(mine.cpu().numpy(), ref) <= GRAD_TOL
    # no gradient reaches the first value row of a sequence, nor crosses sequences
    starts = [int(s) for s, l in zip(cu_np[:-1], lengths) if l > 0]
    assert torch.all(dv[starts] == 0)


def test_equal_length_packed_equals_dense_batch(cabi):
    B, T, H, D, Hv, Dv, W = 3, 70, 2, 4, 1, 4, 9
    q = nonzero_randn((B * T, H, D), 61).to(DEV)
    k = nonzero_randn((B * T, H, D), 62).to(DEV)
    v = nonzero_randn((B * T, Hv, Dv), 63).to(DEV)
    go = nonzero_randn((B * T, H, Dv), 64).to(DEV)
    cu = torch.arange(B + 1, dtype=torch.int32, device=DEV) * T
    dense = _run_cabi(cabi, q, k, v, go, (B, T), W, 1.0, 0.2, 3.0, 99)
    packed = _run_cabi(cabi, q, k, v, go, cu, W, 1.0, 0.2, 3.0, 99)
    assert torch.equal(dense[0], packed[0])
    assert torch.equal(dense[1].permute(1, 0, 2).reshape(H, B * T), packed[1])
    for a, b in zip(dense[4:], packed[4:]):
        assert torch.equal(a, b)


def test_invalid_offsets_set_status_and_zero_outputs(cabi):
    N, H, D, Dv = 20, 2, 3, 4
    q = nonzero_randn((N, H, D), 71).to(DEV)
    v = nonzero_randn((N, 1, Dv), 72).to(DEV)
    for offsets, status in (([1, 10, 20], 1), ([0, 12, 8, 20], 2), ([0, 10, 19], 3)):
        cu = torch.tensor(offsets, dtype=torch.int32, device=DEV)
        out, pq, pk, routes, ws = cabi.hard_forward(q, q, v, cu, 8)
        assert cabi.read_status(ws) == status
        assert not out.any() and torch.all(routes == -1)
    cu = torch.tensor([0, 10, 20], dtype=torch.int32, device=DEV)
    out, pq, pk, routes, ws = cabi.hard_forward(q, q, v, cu, 8)
    assert cabi.read_status(ws) == 0


def test_dropout_shard_offsets_reproduce_unsharded_masks(cabi):
    """Sharding by (batch x value-head group): each shard passes its global coordinates."""
    B, T, H, D, Hv, Dv, W = 2, 80, 4, 4, 2, 4, 8
    q = nonzero_randn((B * T, H, D), 81).to(DEV)
    k = nonzero_randn((B * T, H, D), 82).to(DEV)
    v = nonzero_randn((B * T, Hv, Dv), 83).to(DEV)
    go = nonzero_randn((B * T, H, Dv), 84).to(DEV)
    full = _run_cabi(cabi, q, k, v, go, (B, T), W, 1.0, 0.3, 3.0, 4242)
    seed_t = torch.tensor(4242, dtype=torch.int64, device=DEV)
    group = H // Hv
    for b in range(B):
        for vh in range(Hv):
            rows = slice(b * T, (b + 1) * T)
            hs = slice(vh * group, (vh + 1) * group)
            qs, ks = q[rows, hs].contiguous(), k[rows, hs].contiguous()
            vs, gs = v[rows, vh:vh + 1].contiguous(), go[rows, hs].contiguous()
            out, pq, pk, _, _ = cabi.hard_forward(qs, ks, vs, (1, T), W, want_routes=False)
            dq, dk, dv, _ = cabi.surrogate_vjp(qs, ks, vs, gs, (1, T), pq, pk, W, 1.0, 0.3, 3.0,
                                               seed_t, 7, batch_offset=b, head_offset=vh * group)
            assert torch.equal(out, full[0][rows, hs])
            assert torch.equal(dq, full[4][rows, hs])
            assert torch.equal(dk, full[5][rows, hs])
            assert torch.equal(dv, full[6][rows, vh:vh + 1])


def test_hard_inference_against_oracle_and_reference_fixture(cabi):
    from oracle import rosa_oracle as orc
    z = np.load(os.path.join(GOLDEN, "runtime_cases.npz"))
    for c in range(int(z["n"])):
        cu_np, W = z[f"c{c}_cu"], int(z[f"c{c}_W"])
        qs = torch.from_numpy(z[f"c{c}_q"].astype(np.int32)).to(DEV)
        ks = torch.from_numpy(z[f"c{c}_k"].astype(np.int32)).to(DEV)
        pay = torch.from_numpy(z[f"c{c}_payload"].astype(np.float32))[:, :, None].contiguous().to(DEV)
        cu = torch.from_numpy(cu_np.astype(np.int32)).to(DEV)
        out, end, _ = cabi.hard_inference(qs, ks, pay, cu, W)
        assert np.array_equal(end.cpu().numpy(), z[f"c{c}_end"])
        assert np.array_equal(out[:, :, 0].cpu().numpy().astype(np.uint8), z[f"c{c}_out"])
    # 32-bit symbols with planted copies, dense streams
    rng = np.random.default_rng(7)
    streams, T, H, Hp, Dp, W = 3, 1300, 4, 2, 8, 48
    q = rng.integers(0, 1 << 32, size=(streams, T, H), dtype=np.uint64).astype(np.uint32)
    k = rng.integers(0, 1 << 32, size=(streams, T, H), dtype=np.uint64).astype(np.uint32)
    for s in range(streams):
        for _ in range(12):
            length = int(rng.integers(8, 120))
            src = int(rng.integers(0, T - 2 * length - 2))
            dst = int(rng.integers(src + length, T - length))
            q[s, dst:dst + length] = k[s, src:src + length]
    pay = rng.standard_normal((streams, T, Hp, Dp)).astype(np.float32)
    flat = lambda a: a.reshape((streams * T,) + a.shape[2:])
    cu_np = np.arange(streams + 1, dtype=np.int64) * T
    ref_out, ref_end = orc.hard_inference(flat(q), flat(k), flat(pay), cu_np, W)
    out, end, _ = cabi.hard_inference(torch.from_numpy(flat(q).view(np.int32)).to(DEV),
                                      torch.from_numpy(flat(k).view(np.int32)).to(DEV),
                                      torch.from_numpy(flat(pay)).to(DEV), (streams, T), W)
    assert np.array_equal(end.cpu().numpy(), ref_end)
    assert np.array_equal(out.cpu().numpy(), ref_out)
    assert (ref_end >= 0).mean() > 0.1


# ---------------------------------------------------------------- torch operator surface

def test_public_operator_matches_fixture_and_casts(ops):
    z = np.load(os.path.join(GOLDEN, "dense_bf16_grouped.npz"))
    dev = lambda a: torch.from_numpy(a.astype(np.float32)).to(DEV, torch.bfloat16)
    q, k, v, go = dev(z["q"]), dev(z["k"]), dev(z["v"]), dev(z["go"])
    ql, kl, vl = (t.clone().requires_grad_(True) for t in (q, k, v))
    # explicit seed through the registered operator (the public wrapper draws its own)
    out, pq, pk = torch.ops.rosa_soft.hard_forward(ql, kl, vl, int(z["W"]))
    assert out.dtype == torch.bfloat16 and pq.shape == (q.shape[0], q.shape[2], q.shape[1])
    assert pq.stride() == (q.shape[2] * q.shape[1], q.shape[1], 1)
    seed = torch.tensor(int(z["dropout_seed"]), dtype=torch.int64, device=DEV)
    dq, dk, dv = torch.ops.rosa_soft.surrogate_vjp_masked(
        q, k, v, go, pq, pk, seed, int(z["W"]), float(z["scale"]), float(z["p"]), float(z["m"]), 7)
    assert dq.dtype == torch.float32
    assert np.array_equal(out.detach().float().cpu().numpy(), z["out"])
    for mine, ref in ((dq, z["dq"]), (dk, z["dk"]), (dv, z["dv"])):
        assert normalised_error(mine.to(torch.bfloat16).float().cpu().numpy(), ref) <= 2e-2


def test_public_autograd_path_and_rng_contract(ops):
    B, T, H, D, Hv, Dv = 2, 50, 2, 4, 1, 3
    q = nonzero_randn((B, T, H, D), 91).to(DEV).requires_grad_(True)
    k = nonzero_randn((B, T, H, D), 92).to(DEV).requires_grad_(True)
    v = nonzero_randn((B, T, Hv, Dv), 93).to(DEV).requires_grad_(True)
    # no RNG is consumed without dropout or without grad
    torch.cuda.manual_seed(5)
    state = torch.cuda.get_rng_state()
    ops.rosa_soft(q, k, v, max_suffix_length=8).sum().backward()
    with torch.no_grad():
        ops.rosa_soft(q, k, v, max_suffix_length=8, dropout_p=0.3)
    assert torch.equal(state, torch.cuda.get_rng_state())
    # seeded dropout is reproducible and differs from the no-dropout gradient
    grads = []
    for _ in range(2):
        torch.cuda.manual_seed(123)
        for t in (q, k, v):
            t.grad = None
        out = ops.rosa_soft(q, k, v, max_suffix_length=8, dropout_p=0.3)
        out.backward(torch.ones_like(out))
        grads.append([t.grad.clone() for t in (q, k, v)])
    for a, b in zip(*grads):
        assert torch.equal(a, b)
    # masked-off inputs get no gradient
    q2 = q.detach().clone()
    out = ops.rosa_soft(q2, k, v, max_suffix_length=8)
    out.sum().backward()
    assert q2.grad is None
    # must not raise in deterministic mode: the backward reduces in a fixed order
    torch.use_deterministic_algorithms(True)
    try:
        ops.rosa_soft(q, k, v, max_suffix_length=8).sum().backward()
    finally:
        torch.use_deterministic_algorithms(False)


def test_public_varlen_and_non_contiguous_inputs(ops):
    lengths = [3, 0, 5, 2, 40]
    N, H, D, Hv, Dv = sum(lengths), 2, 3, 1, 4
    cu_np = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)
    base = nonzero_randn((N, H, 2 * D), 95).to(DEV)
    q = base[..., ::2].requires_grad_(True)       # strided view
    k = nonzero_randn((N, H, D), 96).to(DEV).requires_grad_(True)
    v = nonzero_randn((N, Hv, Dv), 97).to(DEV).requires_grad_(True)
    cu_wide = torch.zeros(2 * len(cu_np), dtype=torch.int32, device=DEV)
    cu_wide[::2] = torch.from_numpy(cu_np.astype(np.int32)).to(DEV)
    cu = cu_wide[::2]                              # non-contiguous offsets
    out = ops.rosa_soft_varlen(q, k, v, cu, max_suffix_length=6)
    go = nonzero_randn((N, H, Dv), 98).to(DEV)
    out.backward(go)
    ref_out, _ = oracle_forward(q, k, v, cu_np, 6)
    assert np.array_equal(out.detach().cpu().numpy(), ref_out)
    rq, rk, rv = oracle_grads(q, k, v, go, cu_np, 6, 1.0, 0.0, 3.0, 0)
    assert normalised_error(q.grad.cpu().numpy(), rq) <= GRAD_TOL
    assert normalised_error(k.grad.cpu().numpy(), rk) <= GRAD_TOL
    assert normalised_error(v.grad.cpu().numpy(), rv) <= GRAD_TOL


def test_torch_compile_aot_eager_fullgraph(ops):
    B, T, H, D, Hv, Dv = 1, 40, 2, 4, 1, 3
    q = nonzero_randn((B, T, H, D), 101).to(DEV).requires_grad_(True)
    k = nonzero_randn((B, T, H, D), 102).to(DEV).requires_grad_(True)
    v = nonzero_randn((B, T, Hv, Dv), 103).to(DEV).requires_grad_(True)

    def fn(q, k, v):
        return ops.rosa_soft(q, k, v, max_suffix_length=8, dropout_p=0.1)

    compiled = torch.compile(fn, backend="aot_eager", fullgraph=True)
    torch.cuda.manual_seed(3)
    out = compiled(q, k, v)
    out.backward(torch.ones_like(out))
    got = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    torch.cuda.manual_seed(3)
    eager = fn(q, k, v)
    eager.backward(torch.ones_like(eager))
    assert torch.equal(out, eager)
    for a, t in zip(got, (q, k, v)):
        assert torch.equal(a, t.grad)


def test_operator_error_messages(ops):
    q = nonzero_randn((1, 8, 2, 4), 1).to(DEV)
    v = nonzero_randn((1, 8, 1, 3), 2).to(DEV)
    with pytest.raises(TypeError, match="max_suffix_length must be an integer"):
        ops.rosa_soft(q, q, v, max_suffix_length=2.5)
    with pytest.raises(ValueError, match="scale must be finite"):
        ops.rosa_soft(q, q, v, scale=0.0)
    with pytest.raises(ValueError, match="requires CUDA tensors"):
        ops.rosa_soft(q.cpu(), q.cpu(), v.cpu())
    out, pq, pk = torch.ops.rosa_soft.hard_forward(q, q, v, 4)
    empty = torch.empty(0, dtype=torch.int64, device=DEV)
    with pytest.raises(RuntimeError, match="packed_query_symbols head mismatch"):
        torch.ops.rosa_soft.surrogate_vjp_masked(q, q, v, out, pq[:, :1], pk, empty, 4, 1.0, 0.0,
                                                 3.0, 7)
    with pytest.raises(RuntimeError, match="scalar exactly"):
        torch.ops.rosa_soft.surrogate_vjp_masked(q, q, v, out, pq, pk, empty, 4, 1.0, 0.5, 3.0, 7)
    with pytest.raises(RuntimeError, match=r"gradient_mask must be an integer bit mask in \[1, 7\]"):
        torch.ops.rosa_soft.surrogate_vjp_masked(q, q, v, out, pq, pk, empty, 4, 1.0, 0.0, 3.0, 0)


def test_route_inspection_matches_oracle_dense_and_packed():
    """Selected routes and winning match lengths come out of the forward's own winners
    (reference: selected_route_indices / exact_suffix_lengths of rosa_soft/testing.py:49-117)."""
    import rosa_soft_b200 as rs
    from oracle import rosa_oracle as orc
    B, T, H, D, Hv, Dv, W = 2, 333, 4, 2, 2, 8, 24
    q = nonzero_randn((B, T, H, D), 1, torch.float32)
    k = torch.where(torch.rand(B, T, H, D, generator=torch.Generator().manual_seed(3)) < 0.8, q, -q)
    v = nonzero_randn((B, T, Hv, Dv), 2, torch.float32)
    flat = lambda t: t.reshape(B * T, *t.shape[2:]).numpy()
    cu = np.arange(B + 1) * T
    qs, ks = orc.pack_symbols(flat(q)), orc.pack_symbols(flat(k))
    want_route, want_len = orc.hard_routes(qs, ks, cu, W)
    want_out, _ = orc.hard_forward(flat(q), flat(k), flat(v), cu, W)
    out, info = rs.inspect_hard_routes(q.to(DEV), k.to(DEV), v.to(DEV), max_suffix_length=W)
    assert info.selected_route_indices.shape == (B, H, T) and info.effective_max_suffix_length == W
    got_route = info.selected_route_indices.permute(0, 2, 1).reshape(B * T, H).cpu().numpy()
    got_len = info.selected_match_lengths.permute(0, 2, 1).reshape(B * T, H).cpu().numpy()
    assert np.array_equal(got_route, want_route) and np.array_equal(got_len, want_len)
    assert np.array_equal(out.reshape(B * T, H, Dv).cpu().numpy(), want_out)
    assert (got_len[got_route == 0] == 0).all() and got_len.max() <= W
    assert 0.0 <= info.null_route_fraction < 1.0 and info.mean_match_length >= 1.0
    # packed: ragged sequences with an empty one
    lengths = [100, 0, 233, 1, 332]
    cu_p = np.concatenate([[0], np.cumsum(lengths)])
    want_route, want_len = orc.hard_routes(qs, ks, cu_p, W)
    _, info = rs.inspect_hard_routes(q.reshape(B * T, H, D).to(DEV), k.reshape(B * T, H, D).to(DEV),
                                     v.reshape(B * T, Hv, Dv).to(DEV),
                                     torch.from_numpy(cu_p.astype(np.int32)).to(DEV),
                                     max_suffix_length=W)
    assert np.array_equal(info.selected_route_indices.t().cpu().numpy(), want_route)
    assert np.array_equal(info.selected_match_lengths.t().cpu().numpy(), want_len)
    # route statistics of the packed case against their definitions on the oracle's routes
    # (reference: hard_nonnull_route_fraction / hard_route_lag_mean of
    # rosa_soft/diagnostics.py:264-274, _symbol_health of diagnostics.py:186-207)
    qp, kp = q.reshape(B * T, H, D), k.reshape(B * T, H, D)
    diag = rs.summarize_hard_routes(info, qp.to(DEV), kp.to(DEV))
    rows = np.concatenate([np.arange(n) for n in lengths])
    hit = want_route > 0
    assert abs(diag.hard_nonnull_route_fraction - hit.mean()) < 1e-6
    assert abs(diag.hard_route_lag_mean - (rows[:, None] - want_route)[hit].mean()) < 1e-4
    assert abs(diag.selected_match_length_mean - want_len[hit].mean()) < 1e-4
    assert abs(diag.horizon_hit_fraction - (want_len[hit] >= W).mean()) < 1e-6
    assert abs(diag.query.positive_fraction - float((qp > 0).float().mean())) < 1e-6
    assert abs(diag.key.sign_margin_low_quantile - float(torch.quantile(kp.abs().reshape(-1), 0.05))) < 1e-5
    assert abs(diag.key.softsign_derivative_mean
               - float((1.0 + kp.abs()).square().reciprocal().mean())) < 1e-6


def test_hard_inference_with_a_horizon_beyond_the_narrow_key_range(cabi):
    """A horizon of 2500 with one copied stretch of 2600 symbols: the match length passes 2047
    (beyond the 11-bit length field of the narrow candidate keys).  Each row has a single genuine
    candidate, so the hashed prefilter resolves it by walking the match backwards; the generic
    run-length matcher is covered by the constant-stream case of test_gpu_parity_wide.py."""
    from oracle import rosa_oracle as orc
    rng = np.random.default_rng(17)
    T, H, Hp, Dp, W = 6000, 2, 1, 4, 2500
    k = rng.integers(0, 1 << 32, size=(T, H), dtype=np.uint64).astype(np.uint32)
    q = rng.integers(0, 1 << 32, size=(T, H), dtype=np.uint64).astype(np.uint32)
    q[3200:5800] = k[100:2700]            # rows 3200.. match keys 100.. for 2600 steps
    q[700:760, 1] = k[650:710, 1]
    pay = rng.standard_normal((T, Hp, Dp)).astype(np.float32)
    cu_np = np.array([0, T], dtype=np.int64)
    ref_out, ref_end = orc.hard_inference(q, k, pay, cu_np, W)
    out, end, _ = cabi.hard_inference(torch.from_numpy(q.view(np.int32)).to(DEV),
                                      torch.from_numpy(k.view(np.int32)).to(DEV),
                                      torch.from_numpy(pay).to(DEV), (1, T), W)
    assert np.array_equal(end.cpu().numpy(), ref_end)
    assert np.array_equal(out.cpu().numpy(), ref_out)
    assert int((ref_end[5799] >= 0).sum()) == H      # the long copy really is matched
