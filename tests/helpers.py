"""Shared helpers of the GPU parity tests (seeded inputs, oracle calls, error metrics)."""
from __future__ import annotations

import numpy as np
import torch

from oracle import rosa_oracle as orc

TORCH_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
                "float64": torch.float32}


def nonzero_randn(shape, seed, dtype=torch.float32):
    """|x| >= 0.2 so that signs are unambiguous in every dtype (same construction as the
    reference tests, tests/test_soft_cuda.py:18-26)."""
    g = torch.Generator().manual_seed(seed)
    values = torch.randn(shape, dtype=torch.float32, generator=g)
    values = values.sign().masked_fill(values == 0, 1) * (values.abs() + 0.2)
    return values.to(dtype)


def repeated_stream_logits(n_tokens, heads, bits, seed, repeat_prob=0.3, seg=(4, 40), scale=0.7):
    """+-scale logits of a token stream over alphabet 2**bits in which segments repeat, so hard
    matches are long (the long-match stress construction)."""
    rng = np.random.default_rng(seed)
    out = np.empty((n_tokens, heads, bits), np.float32)
    for h in range(heads):
        toks = []
        while len(toks) < n_tokens:
            length = int(rng.integers(seg[0], seg[1] + 1))
            if toks and rng.random() < repeat_prob and len(toks) > length:
                start = int(rng.integers(0, len(toks) - length + 1))
                toks.extend(toks[start:start + length])
            else:
                toks.extend(rng.integers(0, 1 << bits, size=length).tolist())
        toks = np.array(toks[:n_tokens])
        for d in range(bits):
            out[:, h, d] = np.where((toks >> d) & 1, scale, -scale)
    return torch.from_numpy(out)


def normalised_error(mine, ref):
    ref = np.asarray(ref, dtype=np.float64)
    mine = np.asarray(mine, dtype=np.float64).reshape(ref.shape)
    scale = max(float(np.abs(ref).max()), 1e-30)
    return float(np.abs(mine - ref).max()) / scale


def oracle_grads(q, k, v, go, cu, W, scale, p, m, seed, mask=7, batch_offset=0):
    f = lambda t: t.detach().float().cpu().numpy()
    return orc.surrogate_vjp(f(q), f(k), f(v), f(go), cu, W, scale, p, m, seed, batch_offset, mask)


def oracle_forward(q, k, v, cu, W):
    f = lambda t: t.detach().float().cpu().numpy()
    return orc.hard_forward(f(q), f(k), f(v), cu, W)


# element-wise bound |mine - ref| <= rtol * |ref| + atol_frac * max|ref| per input dtype; the half
# types are compared after the cast to the input dtype, with the reference's own tolerances
CLOSE_RTOL = {"float64": 1e-4, "float32": 1e-4, "bfloat16": 2e-2, "float16": 3e-3}
CLOSE_ATOL_FRAC = {"float64": 2e-5, "float32": 2e-5, "bfloat16": 4e-3, "float16": 1e-3}


def assert_grads_close(mine, ref, dtype_name, label=""):
    """allclose-style check of a float32 gradient tensor against a reference array."""
    ref = np.asarray(ref, dtype=np.float64)
    if dtype_name in ("bfloat16", "float16"):
        mine = mine.to(TORCH_DTYPES[dtype_name]).float()
    got = mine.detach().cpu().numpy().astype(np.float64).reshape(ref.shape)
    bound = CLOSE_RTOL[dtype_name] * np.abs(ref) + CLOSE_ATOL_FRAC[dtype_name] * np.abs(ref).max()
    excess = np.abs(got - ref) - bound
    worst = int(np.argmax(excess))
    assert excess.max() <= 0, (label, "element", worst, "got", got.reshape(-1)[worst], "want",
                               ref.reshape(-1)[worst], "bound", bound.reshape(-1)[worst])


# Normalised max error allowed for the operator's float32 gradients against the float64 oracle, by
# input dtype.  float32 inputs: the operator contract's 1e-4.  Half-precision inputs are held to
# 3e-3 / 2e-2 only AFTER the cast to the input dtype by the contract; the float32 outputs are
# checked much tighter than that here: the bound is what the bf16 operand terms of the tensor-core
# contraction keep (float16: two terms of every operand; bfloat16: one term of p*d, 8 bits).
GRAD_TOL_BY_DTYPE = {torch.float32: 1e-4, torch.float16: 2e-4, torch.bfloat16: 4e-3}


def grad_tol(dtype):
    return GRAD_TOL_BY_DTYPE[dtype]
