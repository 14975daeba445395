"""Generate golden input/output vectors by running the UNMODIFIED reference.

Run in a container where the reference tree is mounted, with ``$ROSA_REFERENCE_ROOT`` naming
its root:  ``ROSA_REFERENCE_ROOT=<reference checkout> python tests/golden/make_golden.py``.
It imports ``rosa_soft`` from that tree (pure-PyTorch ``reference`` variant, CPU)
and, when ``oracle/_ref/librosa_runtime_ref.so`` has been built by
``oracle/build_ref.py``, the reference's own RosaRuntime.  The ``.npz`` files it
writes next to this script are committed; the tests never need the reference.

Every case stores its inputs (float32 arrays holding exactly the values of the
case dtype), the controls, and the reference's outputs: hard output, selected
routes from ``rosa_soft.testing.inspect_rosa_soft`` and the gradients returned
by autograd through ``rosa_soft_reference`` / ``rosa_soft_varlen_reference``.
"""
from __future__ import annotations

import os
import sys

sys.dont_write_bytecode = True
REFERENCE_ROOT = os.environ.get("ROSA_REFERENCE_ROOT")
if not REFERENCE_ROOT or not os.path.isdir(os.path.join(REFERENCE_ROOT, "rosa_soft")):
    raise SystemExit("set ROSA_REFERENCE_ROOT to the root of the reference checkout")
sys.path.insert(0, REFERENCE_ROOT)

import numpy as np
import torch

import rosa_soft
from rosa_soft.soft_reference import (
    _apply_attention_dropout,
    _hash_dropout_counter,
    _rosa_soft_reference_with_seed,
)
from rosa_soft.testing import inspect_rosa_soft

HERE = os.path.dirname(os.path.abspath(__file__))
DTYPES = {"float64": torch.float64, "float32": torch.float32, "bfloat16": torch.bfloat16,
          "float16": torch.float16}


def nonzero_randn(shape, seed, dtype):
    """Same construction as the reference tests' helper (tests/test_soft_cuda.py:18-26)."""
    g = torch.Generator().manual_seed(seed)
    values = torch.randn(shape, dtype=torch.float32, generator=g)
    values = values.sign().masked_fill(values == 0, 1) * (values.abs() + 0.2)
    return values.to(dtype)


def f32(t):
    return t.detach().to(torch.float64 if t.dtype == torch.float64 else torch.float32).numpy()


def dense_case(name, B, T, H, D, Hv, Dv, W, scale, p, m, dtype, seed, mode="randn", loss="random",
               dropout_seed=None):
    dt = DTYPES[dtype]
    if mode == "randn":
        q = nonzero_randn((B, T, H, D), seed, dt)
        k = nonzero_randn((B, T, H, D), seed + 1, dt)
    elif mode == "allmatch":
        q = nonzero_randn((B, T, H, D), seed, dt).abs()
        k = nonzero_randn((B, T, H, D), seed + 1, dt).abs()
        k[:, T // 3, :, 0] *= -1
    elif mode == "periodic":
        g = torch.Generator().manual_seed(seed)
        base = torch.randint(0, 2, (B, 5, H, D), generator=g).float() * 2 - 1
        reps = (T + 4) // 5
        q = (base.repeat(1, reps, 1, 1)[:, :T] * 0.7).to(dt)
        k = q.clone()
    elif mode == "repeat":
        # token stream over alphabet 2^D in which earlier segments are copied: long exact matches
        rng = np.random.default_rng(seed)
        logits = np.empty((B, T, H, D), np.float32)
        for b in range(B):
            for h in range(H):
                toks = []
                while len(toks) < T:
                    n = int(rng.integers(4, 25))
                    if toks and rng.random() < 0.4 and len(toks) > n:
                        a = int(rng.integers(0, len(toks) - n + 1))
                        toks.extend(toks[a:a + n])
                    else:
                        toks.extend(rng.integers(0, 1 << D, size=n).tolist())
                toks = np.array(toks[:T])
                logits[b, :, h, :] = np.where((toks[:, None] >> np.arange(D)) & 1, 0.7, -0.7)
        q = torch.from_numpy(logits).to(dt)
        k = q.clone()
    v = nonzero_randn((B, T, Hv, Dv), seed + 2, dt)
    out_ref, insp = inspect_rosa_soft(q, k, v, max_suffix_length=W, scale=scale, dropout_p=0.0,
                                      mismatch_scale=m)
    if loss == "random":
        go = nonzero_randn((B, T, H, Dv), seed + 3, dt)
    else:  # loss = mean(out^2): grad = 2 out / numel
        go = (2.0 * out_ref.to(torch.float32) / out_ref.numel()).to(dt)
    ql, kl, vl = (t.clone().requires_grad_(True) for t in (q, k, v))
    if p > 0:
        sd = torch.tensor(dropout_seed, dtype=torch.int64)
    else:
        sd = torch.empty(0, dtype=torch.int64)
    weff = min(W, T)
    outs = []
    for b in range(B):  # one batch element at a time with its global dropout coordinate
        outs.append(_rosa_soft_reference_with_seed(ql[b:b + 1], kl[b:b + 1], vl[b:b + 1], sd, weff,
                                                   scale, p, m, b))
    out = torch.cat(outs, 0)
    out.backward(go)
    assert torch.equal(out.detach(), out_ref)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        kind="dense", dtype=dtype, W=W, scale=scale, p=p, m=m,
        dropout_seed=np.int64(dropout_seed if p > 0 else 0),
        q=f32(q), k=f32(k), v=f32(v), go=f32(go), out=f32(out),
        routes=insp.selected_route_indices.numpy().astype(np.int32),  # [B,H,T]
        dq=f32(ql.grad), dk=f32(kl.grad), dv=f32(vl.grad),
    )
    print("wrote", name)


def nonfinite_case(name):
    """Infinities, NaN and signed zeros in every input (the policy the reference pins in
    tests/test_soft_cuda.py:570-611): sign bits treat +0, -0 and NaN as "not positive", the
    softsign Jacobian sends +-inf to a zero gradient and NaN to NaN."""
    inf, nan = float("inf"), float("nan")
    q = torch.tensor([[[[inf, -0.5]], [[0.4, -inf]], [[nan, -1.0]], [[0.0, 0.3]], [[-0.0, 0.3]],
                       [[0.7, 0.3]], [[-0.2, 0.9]]]])
    k = torch.tensor([[[[-1.0, inf]], [[-inf, -0.7]], [[0.2, 0.3]], [[-0.0, 0.5]], [[0.0, 0.3]],
                       [[0.6, 0.1]], [[nan, 0.4]]]])
    v = torch.tensor([[[[inf, -1.0]], [[-inf, 0.2]], [[0.5, -0.4]], [[0.0, nan]], [[-0.0, 1.0]],
                       [[0.3, -0.3]], [[1.5, 0.25]]]])
    W, scale, m = 3, 1.0, 3.0
    out_ref, insp = inspect_rosa_soft(q, k, v, max_suffix_length=W, scale=scale, dropout_p=0.0,
                                      mismatch_scale=m)
    go = nonzero_randn((1, 7, 1, 2), 60, torch.float32)
    ql, kl, vl = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = rosa_soft.rosa_soft_reference(ql, kl, vl, max_suffix_length=W, scale=scale, mismatch_scale=m)
    out.backward(go)
    assert torch.equal(out.detach(), out_ref)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        kind="nonfinite", dtype="float32", W=W, scale=scale, p=0.0, m=m, dropout_seed=np.int64(0),
        q=f32(q), k=f32(k), v=f32(v), go=f32(go), out=f32(out),
        routes=insp.selected_route_indices.numpy().astype(np.int32),
        dq=f32(ql.grad), dk=f32(kl.grad), dv=f32(vl.grad),
    )
    print("wrote", name)


def varlen_case(name, lengths, H, D, Hv, Dv, W, scale, p, m, dtype, seed, dropout_seed=None):
    dt = DTYPES[dtype]
    N = sum(lengths)
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    q = nonzero_randn((N, H, D), seed, dt)
    k = nonzero_randn((N, H, D), seed + 1, dt)
    v = nonzero_randn((N, Hv, Dv), seed + 2, dt)
    go = nonzero_randn((N, H, Dv), seed + 3, dt)
    ql, kl, vl = (t.clone().requires_grad_(True) for t in (q, k, v))
    sd = torch.tensor(dropout_seed, dtype=torch.int64) if p > 0 else torch.empty(0, dtype=torch.int64)
    weff = min(W, N)
    outs, routes = [], []
    for s, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        if a == b:
            continue
        outs.append(_rosa_soft_reference_with_seed(ql[a:b][None], kl[a:b][None], vl[a:b][None], sd,
                                                   weff, scale, p, m, s)[0])
        _, insp = inspect_rosa_soft(q[a:b][None], k[a:b][None], v[a:b][None], max_suffix_length=weff)
        routes.append(insp.selected_route_indices[0].T)  # [len, H]
    out = torch.cat(outs, 0)
    out.backward(go)
    # the public varlen oracle must agree when there is no dropout
    if p == 0:
        pub = rosa_soft.rosa_soft_varlen_reference(q, k, v, torch.from_numpy(cu), max_suffix_length=W,
                                                   scale=scale, mismatch_scale=m)
        assert torch.equal(pub, out.detach())
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        kind="varlen", dtype=dtype, W=W, scale=scale, p=p, m=m,
        dropout_seed=np.int64(dropout_seed if p > 0 else 0), cu_seqlens=cu,
        q=f32(q), k=f32(k), v=f32(v), go=f32(go), out=f32(out),
        routes=torch.cat(routes, 0).numpy().astype(np.int32),  # [N,H] local route index
        dq=f32(ql.grad), dk=f32(kl.grad), dv=f32(vl.grad),
    )
    print("wrote", name)


def dropout_kats():
    seeds = [7, (1 << 32) + 7, (1 << 62) + 12345]
    masks = []
    for seed, off in zip(seeds, (0, 3, 11)):
        w = _apply_attention_dropout(torch.ones(2, 3, 9, 9), 0.5, torch.tensor(seed), off)
        masks.append((w > 0).numpy())
    counters = np.array([0, 1, 2, 0xFFFFFFFF, 0x12345678], dtype=np.int64)
    hashed = _hash_dropout_counter(torch.from_numpy(counters)).numpy()
    np.savez_compressed(os.path.join(HERE, "dropout_kats.npz"), seeds=np.array(seeds, dtype=np.int64),
                        offsets=np.array([0, 3, 11]), masks=np.stack(masks), counters=counters,
                        hashed=hashed, p=0.5)
    print("wrote dropout_kats")


def runtime_cases():
    lib = os.path.join(os.path.dirname(os.path.dirname(HERE)), "oracle", "_ref", "librosa_runtime_ref.so")
    if not os.path.exists(lib):
        print("reference runtime not built; skipping runtime cases")
        return
    torch.classes.load_library(lib)
    rng = np.random.default_rng(2024)
    cases = {}
    for idx, (slots, T, H, Hp, bits, W) in enumerate([(3, 97, 4, 2, 1, 5), (2, 300, 2, 2, 2, 32),
                                                      (4, 64, 3, 1, 8, 2), (1, 513, 2, 1, 3, 600)]):
        lengths = rng.integers(T // 2, T + 1, size=slots)
        cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)
        N = int(cu[-1])
        q = rng.integers(0, 1 << bits, size=(N, H), dtype=np.uint8)
        k = rng.integers(0, 1 << bits, size=(N, H), dtype=np.uint8)
        # plant copies so long matches exist
        for s in range(slots):
            a, b = cu[s], cu[s + 1]
            if b - a > 40:
                k[a + 20:a + 35] = k[a:a + 15]
                q[a + 21:a + 36] = k[a + 1:a + 16]
        pay = rng.integers(0, 256, size=(N, Hp), dtype=np.uint8)
        rt = torch.classes.rosa_soft.RosaRuntime(H, Hp, bits, 8, W)
        out, end = rt.update_packed(torch.from_numpy(cu), torch.from_numpy(q), torch.from_numpy(k),
                                    torch.from_numpy(pay))
        cases[f"c{idx}_cu"] = cu
        cases[f"c{idx}_q"] = q
        cases[f"c{idx}_k"] = k
        cases[f"c{idx}_payload"] = pay
        cases[f"c{idx}_out"] = out.numpy()
        cases[f"c{idx}_end"] = end.numpy()
        cases[f"c{idx}_W"] = W
    np.savez_compressed(os.path.join(HERE, "runtime_cases.npz"), n=4, **cases)
    print("wrote runtime_cases")


def main():
    assert rosa_soft.BUILD_CAPABILITIES.variant == "reference"
    torch.set_num_threads(os.cpu_count())
    dense_case("dense_f64_small", 2, 19, 4, 3, 2, 5, 6, 1.3, 0.0, 2.0, "float64", 100)
    dense_case("dense_f64_dropout", 2, 17, 2, 4, 1, 3, 5, 0.8, 0.3, 3.0, "float64", 110,
               dropout_seed=(1 << 33) + 77)
    dense_case("dense_f64_allmatch", 1, 40, 2, 2, 2, 3, 4, 1.0, 0.1, 3.0, "float64", 120,
               mode="allmatch", dropout_seed=991)
    dense_case("dense_f64_periodic_w64", 1, 48, 1, 2, 1, 3, 64, 1.0, 0.0, 3.0, "float64", 130,
               mode="periodic")
    dense_case("dense_f64_w1", 1, 33, 2, 1, 1, 2, 1, 2.0, 0.0, 1.5, "float64", 140, mode="allmatch")
    dense_case("dense_f32_d32_t137", 1, 137, 2, 32, 1, 5, 200, 1.0, 0.0, 3.0, "float32", 150)
    dense_case("dense_f32_config1", 1, 256, 4, 4, 4, 8, 32, 1.0, 0.0, 3.0, "float32", 1001,
               loss="mean_sq")
    dense_case("dense_bf16_grouped", 2, 65, 6, 8, 3, 8, 16, 1.0, 0.1, 3.0, "bfloat16", 160,
               dropout_seed=424242)
    dense_case("dense_f16_small", 1, 70, 4, 5, 2, 6, 9, 1.0, 0.05, 9.0, "float16", 170,
               dropout_seed=5)
    dense_case("dense_f32_t1", 2, 1, 2, 3, 1, 2, 4, 1.0, 0.0, 3.0, "float32", 180)
    # value rows of 9..32 components (the widths of the long-match and packed benchmark
    # configurations), narrow and wide symbols, with and without dropout and a closing window
    dense_case("dense_f32_repeat_d2_dv16", 1, 96, 2, 2, 2, 16, 12, 1.0, 0.0, 3.0, "float32", 190,
               mode="repeat")
    dense_case("dense_f16_d16_dv32", 1, 72, 4, 16, 1, 32, 64, 1.0, 0.05, 9.0, "float16", 191,
               dropout_seed=31337)
    dense_case("dense_bf16_d20_dv24", 1, 60, 2, 20, 2, 24, 7, 1.3, 0.1, 3.0, "bfloat16", 192,
               dropout_seed=(1 << 35) + 5)
    dense_case("dense_f32_d8_dv12", 2, 50, 2, 8, 1, 12, 9, 0.8, 0.2, 2.0, "float32", 193,
               dropout_seed=77)
    nonfinite_case("nonfinite_f32_policy")
    varlen_case("varlen_f64_empty_segments", (3, 0, 5, 2), 2, 3, 1, 4, 4, 1.0, 0.25, 3.0, "float64", 200,
                dropout_seed=(1 << 40) + 3)
    varlen_case("varlen_f32_edges", (1, 2, 127, 0, 128, 129), 2, 4, 2, 3, 160, 1.0, 0.0, 3.0,
                "float32", 210)
    dropout_kats()
    runtime_cases()


if __name__ == "__main__":
    main()
