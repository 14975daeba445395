"""Public CUDA operators ``rosa_soft`` and ``rosa_soft_varlen``.

Same surface as the reference's ``rosa_soft/soft.py``: validation (:29-100), fake (meta)
kernels for the registered operators so that ``torch.compile(backend="aot_eager",
fullgraph=True)`` traces them (:127-256), an autograd function that saves
``(q, k, v[, cu_seqlens], packed_q, packed_k, seed)`` plus the four controls (:259-414) and
the two public entry points with keyword-only controls (:417-508).  Dense and packed calls
share one autograd function here; it dispatches on whether offsets were given.  The kernels
behind ``torch.ops.rosa_soft.*`` live in ``librosa_soft_b200.so``: there is no CPU or eager
fallback.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor
from torch.autograd.function import once_differentiable

from . import soft_contract as _contract
from .sharding import current_dropout_coordinates as _shard_coordinates
from .soft_contract import (  # noqa: F401  (re-exported like the reference module does)
    ROSA_SOFT_DEFAULT_DROPOUT_P,
    ROSA_SOFT_DEFAULT_MISMATCH_SCALE,
    ROSA_SOFT_DEFAULT_SCALE,
)

__all__ = [
    "ROSA_SOFT_DEFAULT_DROPOUT_P",
    "ROSA_SOFT_DEFAULT_MISMATCH_SCALE",
    "ROSA_SOFT_DEFAULT_SCALE",
    "rosa_soft",
    "rosa_soft_varlen",
]

_OPS = torch.ops.rosa_soft
_CUDA_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


# ------------------------------------------------------------------ fake kernels
def _fake_forward(dense: bool):
    def fake(query, key, value, *rest):
        if dense:     # (B, T, H, D) -> output (B, T, H, Dv), symbols (B, H, T)
            batch, seq, heads = query.shape[:3]
            out_shape, sym_shape = (batch, seq, heads, value.shape[3]), (batch, heads, seq)
        else:         # (N, H, D) -> output (N, H, Dv), symbols (H, N)
            tokens, heads = query.shape[:2]
            out_shape, sym_shape = (tokens, heads, value.shape[2]), (heads, tokens)
        symbols = [query.new_empty(sym_shape, dtype=torch.int32) for _ in range(2)]
        return query.new_empty(out_shape), symbols[0], symbols[1]
    return fake


def _fake_vjp(query, key, value, *rest):
    gradient_mask = rest[-1]
    # float32 gradients in the input's shape; a masked-off gradient is a (0,) placeholder
    return tuple(
        t.new_empty(t.shape if gradient_mask & bit else (0,), dtype=torch.float32)
        for bit, t in ((1, query), (2, key), (4, value))
    )


def _fake_vjp_sharded(query, key, value, cu_seqlens, *rest):
    return _fake_vjp(query, key, value, *rest[:-2])


def _fake_inference(query_symbols, key_symbols, payload, cu_seqlens, max_suffix_length):
    return (payload.new_empty((*query_symbols.shape, payload.shape[-1])),
            query_symbols.new_empty(query_symbols.shape, dtype=torch.int64))


for _name, _fake in (
    ("hard_forward", _fake_forward(dense=True)),
    ("hard_forward_varlen", _fake_forward(dense=False)),
    ("surrogate_vjp_masked", _fake_vjp),
    ("surrogate_vjp_varlen_masked", _fake_vjp),
    ("surrogate_vjp_sharded", _fake_vjp_sharded),
    ("hard_inference", _fake_inference),
):
    torch.library.register_fake(f"rosa_soft::{_name}")(_fake)


# --------------------------------------------------------------- autograd function
class _HardForwardSoftVjp(torch.autograd.Function):
    """Exact hard forward; dense surrogate VJP in backward.  ``cu_seqlens`` is ``None`` for
    a dense batch."""

    @staticmethod
    def forward(ctx, query, key, value, cu_seqlens, dropout_seed, max_suffix_length, scale,
                dropout_p, mismatch_scale):
        horizon = int(max_suffix_length)
        if cu_seqlens is None:
            output, packed_q, packed_k = _OPS.hard_forward(query, key, value, horizon)
            ctx.save_for_backward(query, key, value, packed_q, packed_k, dropout_seed)
        else:
            output, packed_q, packed_k = _OPS.hard_forward_varlen(query, key, value, cu_seqlens,
                                                                  horizon)
            ctx.save_for_backward(query, key, value, packed_q, packed_k, dropout_seed, cu_seqlens)
        ctx.controls = (horizon, float(scale), float(dropout_p), float(mismatch_scale))
        ctx.shard = _shard_coordinates()   # (0, 0) unless inside sharding.dropout_coordinates
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        query, key, value, packed_q, packed_k, dropout_seed, *offsets = ctx.saved_tensors
        wanted = ctx.needs_input_grad[:3]
        mask = sum(bit for bit, need in zip((1, 2, 4), wanted) if need)
        if ctx.shard != (0, 0):
            gradients = _OPS.surrogate_vjp_sharded(query, key, value,
                                                   offsets[0] if offsets else None, grad_output,
                                                   packed_q, packed_k, dropout_seed,
                                                   *ctx.controls, mask, *ctx.shard)
        elif offsets:
            gradients = _OPS.surrogate_vjp_varlen_masked(query, key, value, offsets[0], grad_output,
                                                         packed_q, packed_k, dropout_seed,
                                                         *ctx.controls, mask)
        else:
            gradients = _OPS.surrogate_vjp_masked(query, key, value, grad_output, packed_q,
                                                  packed_k, dropout_seed, *ctx.controls, mask)
        # the operator returns float32; hand autograd the input dtype
        cast = [g.to(t.dtype) if need else None
                for g, t, need in zip(gradients, (query, key, value), wanted)]
        return (*cast, None, None, None, None, None, None)


# ------------------------------------------------------------------- entry points
def _check_cuda_inputs(name: str, query: Tensor, horizon: int, scale, dropout_p, mismatch_scale):
    if not query.is_cuda:
        raise ValueError(f"{name} requires CUDA tensors")
    if query.dtype not in _CUDA_DTYPES:
        raise ValueError(f"{name} supports float32, float16, and bfloat16")
    _contract.validate_fp32_surrogate_scalars(horizon, scale, dropout_p, mismatch_scale)


def _run(query, key, value, cu_seqlens: Optional[Tensor], horizon, scale, dropout_p,
         mismatch_scale):
    trains = torch.is_grad_enabled() and (query.requires_grad or key.requires_grad
                                          or value.requires_grad)
    if not trains:     # inference fast path: no seed is drawn, nothing is saved
        if cu_seqlens is None:
            return _OPS.hard_forward(query, key, value, horizon)[0]
        return _OPS.hard_forward_varlen(query, key, value, cu_seqlens, horizon)[0]
    seed = _contract.make_dropout_seed(query, dropout_p, trains)
    return _HardForwardSoftVjp.apply(query, key, value, cu_seqlens, seed, horizon, float(scale),
                                     float(dropout_p), float(mismatch_scale))


def rosa_soft(query: Tensor, key: Tensor, value: Tensor, *, max_suffix_length: int = 32,
              scale: float = ROSA_SOFT_DEFAULT_SCALE,
              dropout_p: float = ROSA_SOFT_DEFAULT_DROPOUT_P,
              mismatch_scale: float = ROSA_SOFT_DEFAULT_MISMATCH_SCALE) -> Tensor:
    """Run exact hard ROSA forward with a dense attention-style CUDA VJP."""
    horizon = _contract.validate_rosa_soft_inputs(query, key, value, max_suffix_length, scale,
                                                  dropout_p, mismatch_scale)
    _check_cuda_inputs("rosa_soft", query, horizon, scale, dropout_p, mismatch_scale)
    return _run(query, key, value, None, horizon, scale, dropout_p, mismatch_scale)


def rosa_soft_varlen(query: Tensor, key: Tensor, value: Tensor, cu_seqlens: Tensor, *,
                     max_suffix_length: int = 32, scale: float = ROSA_SOFT_DEFAULT_SCALE,
                     dropout_p: float = ROSA_SOFT_DEFAULT_DROPOUT_P,
                     mismatch_scale: float = ROSA_SOFT_DEFAULT_MISMATCH_SCALE) -> Tensor:
    """Run RosaSoft independently over CUDA-packed variable-length sequences."""
    horizon = _contract.validate_rosa_soft_varlen_inputs(query, key, value, cu_seqlens,
                                                         max_suffix_length, scale, dropout_p,
                                                         mismatch_scale)
    _check_cuda_inputs("rosa_soft_varlen", query, horizon, scale, dropout_p, mismatch_scale)
    return _run(query, key, value, cu_seqlens, horizon, scale, dropout_p, mismatch_scale)
