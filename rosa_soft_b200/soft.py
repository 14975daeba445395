"""Public CUDA operators ``rosa_soft`` and ``rosa_soft_varlen``.

Mirrors the reference's ``rosa_soft/soft.py``: validation (:29-100), fake (meta)
registrations of the four operators so that ``torch.compile(backend="aot_eager",
fullgraph=True)`` traces them (:127-256), two ``autograd.Function`` classes that save
``(q, k, v[, cu_seqlens], packed_q, packed_k, seed)`` (:259-414) and the public entry points
with the keyword-only controls (:417-508).  The kernels behind ``torch.ops.rosa_soft.*``
live in ``librosa_soft_b200.so``; there is no CPU or eager fallback.
"""
from __future__ import annotations

import torch
from torch import Tensor
from torch.autograd.function import once_differentiable

from .soft_contract import (
    ROSA_SOFT_DEFAULT_DROPOUT_P,
    ROSA_SOFT_DEFAULT_MISMATCH_SCALE,
    ROSA_SOFT_DEFAULT_SCALE,
    make_dropout_seed,
    validate_fp32_surrogate_scalars,
    validate_rosa_soft_inputs,
    validate_rosa_soft_varlen_inputs,
)

__all__ = [
    "ROSA_SOFT_DEFAULT_DROPOUT_P",
    "ROSA_SOFT_DEFAULT_MISMATCH_SCALE",
    "ROSA_SOFT_DEFAULT_SCALE",
    "rosa_soft",
    "rosa_soft_varlen",
]

_CUDA_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


def _validate_cuda_call(query, key, value, max_suffix_length, scale, dropout_p, mismatch_scale):
    effective = validate_rosa_soft_inputs(query, key, value, max_suffix_length, scale, dropout_p,
                                          mismatch_scale)
    if not query.is_cuda:
        raise ValueError("rosa_soft requires CUDA tensors")
    if query.dtype not in _CUDA_DTYPES:
        raise ValueError("rosa_soft supports float32, float16, and bfloat16")
    validate_fp32_surrogate_scalars(effective, scale, dropout_p, mismatch_scale)
    return effective


def _validate_cuda_varlen_call(query, key, value, cu_seqlens, max_suffix_length, scale, dropout_p,
                               mismatch_scale):
    effective = validate_rosa_soft_varlen_inputs(query, key, value, cu_seqlens, max_suffix_length,
                                                 scale, dropout_p, mismatch_scale)
    if not query.is_cuda:
        raise ValueError("rosa_soft_varlen requires CUDA tensors")
    if query.dtype not in _CUDA_DTYPES:
        raise ValueError("rosa_soft_varlen supports float32, float16, and bfloat16")
    validate_fp32_surrogate_scalars(effective, scale, dropout_p, mismatch_scale)
    return effective


def _gradient_mask(needs_input_grad) -> int:
    needs_query, needs_key, needs_value = needs_input_grad[:3]
    return int(needs_query) | (int(needs_key) << 1) | (int(needs_value) << 2)


def _cast_requested_gradients(gradients, inputs, needs_input_grad):
    return tuple(
        gradient.to(tensor.dtype) if requested else None
        for gradient, tensor, requested in zip(gradients, inputs, needs_input_grad)
    )


def _masked_gradient_fakes(gradient_mask, tensors):
    return tuple(
        t.new_empty(t.shape, dtype=torch.float32) if gradient_mask & bit
        else t.new_empty((0,), dtype=torch.float32)
        for bit, t in zip((1, 2, 4), tensors)
    )


@torch.library.register_fake("rosa_soft::hard_forward")
def _fake_hard_forward(query, key, value, max_suffix_length):
    packed = (query.shape[0], query.shape[2], query.shape[1])
    return (
        query.new_empty((*query.shape[:3], value.shape[3])),
        query.new_empty(packed, dtype=torch.int32),
        query.new_empty(packed, dtype=torch.int32),
    )


@torch.library.register_fake("rosa_soft::hard_forward_varlen")
def _fake_hard_forward_varlen(query, key, value, cu_seqlens, max_suffix_length):
    packed = (query.shape[1], query.shape[0])
    return (
        query.new_empty((*query.shape[:2], value.shape[2])),
        query.new_empty(packed, dtype=torch.int32),
        query.new_empty(packed, dtype=torch.int32),
    )


@torch.library.register_fake("rosa_soft::surrogate_vjp_masked")
def _fake_surrogate_vjp_masked(query, key, value, grad_output, packed_query_symbols,
                               packed_key_symbols, dropout_seed, max_suffix_length, scale,
                               dropout_p, mismatch_scale, gradient_mask):
    return _masked_gradient_fakes(gradient_mask, (query, key, value))


@torch.library.register_fake("rosa_soft::surrogate_vjp_varlen_masked")
def _fake_surrogate_vjp_varlen_masked(query, key, value, cu_seqlens, grad_output,
                                      packed_query_symbols, packed_key_symbols, dropout_seed,
                                      max_suffix_length, scale, dropout_p, mismatch_scale,
                                      gradient_mask):
    return _masked_gradient_fakes(gradient_mask, (query, key, value))


@torch.library.register_fake("rosa_soft::hard_inference")
def _fake_hard_inference(query_symbols, key_symbols, payload, cu_seqlens, max_suffix_length):
    return (
        payload.new_empty((*query_symbols.shape, payload.shape[-1])),
        query_symbols.new_empty(query_symbols.shape, dtype=torch.int64),
    )


class _HardForwardSoftVjpFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, dropout_seed, max_suffix_length, scale, dropout_p,
                mismatch_scale):
        hard_output, packed_q, packed_k = torch.ops.rosa_soft.hard_forward(
            query, key, value, int(max_suffix_length))
        ctx.max_suffix_length = int(max_suffix_length)
        ctx.scale = float(scale)
        ctx.dropout_p = float(dropout_p)
        ctx.mismatch_scale = float(mismatch_scale)
        ctx.save_for_backward(query, key, value, packed_q, packed_k, dropout_seed)
        return hard_output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        query, key, value, packed_q, packed_k, dropout_seed = ctx.saved_tensors
        needs = ctx.needs_input_grad[:3]
        gradients = torch.ops.rosa_soft.surrogate_vjp_masked(
            query, key, value, grad_output, packed_q, packed_k, dropout_seed,
            ctx.max_suffix_length, ctx.scale, ctx.dropout_p, ctx.mismatch_scale,
            _gradient_mask(needs))
        return (*_cast_requested_gradients(gradients, (query, key, value), needs),
                None, None, None, None, None)


class _HardForwardSoftVjpVarlenFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, cu_seqlens, dropout_seed, max_suffix_length, scale,
                dropout_p, mismatch_scale):
        hard_output, packed_q, packed_k = torch.ops.rosa_soft.hard_forward_varlen(
            query, key, value, cu_seqlens, int(max_suffix_length))
        ctx.max_suffix_length = int(max_suffix_length)
        ctx.scale = float(scale)
        ctx.dropout_p = float(dropout_p)
        ctx.mismatch_scale = float(mismatch_scale)
        ctx.save_for_backward(query, key, value, cu_seqlens, packed_q, packed_k, dropout_seed)
        return hard_output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_output):
        query, key, value, cu_seqlens, packed_q, packed_k, dropout_seed = ctx.saved_tensors
        needs = ctx.needs_input_grad[:3]
        gradients = torch.ops.rosa_soft.surrogate_vjp_varlen_masked(
            query, key, value, cu_seqlens, grad_output, packed_q, packed_k, dropout_seed,
            ctx.max_suffix_length, ctx.scale, ctx.dropout_p, ctx.mismatch_scale,
            _gradient_mask(needs))
        return (*_cast_requested_gradients(gradients, (query, key, value), needs),
                None, None, None, None, None, None)


def rosa_soft(query: Tensor, key: Tensor, value: Tensor, *, max_suffix_length: int = 32,
              scale: float = ROSA_SOFT_DEFAULT_SCALE,
              dropout_p: float = ROSA_SOFT_DEFAULT_DROPOUT_P,
              mismatch_scale: float = ROSA_SOFT_DEFAULT_MISMATCH_SCALE) -> Tensor:
    """Run exact hard ROSA forward with a dense attention-style CUDA VJP."""
    max_suffix_length = _validate_cuda_call(query, key, value, max_suffix_length, scale, dropout_p,
                                            mismatch_scale)
    needs_backward = torch.is_grad_enabled() and any(
        t.requires_grad for t in (query, key, value))
    if not needs_backward:
        return torch.ops.rosa_soft.hard_forward(query, key, value, max_suffix_length)[0]
    dropout_seed = make_dropout_seed(query, dropout_p, needs_backward)
    return _HardForwardSoftVjpFunction.apply(query, key, value, dropout_seed, max_suffix_length,
                                             float(scale), float(dropout_p), float(mismatch_scale))


def rosa_soft_varlen(query: Tensor, key: Tensor, value: Tensor, cu_seqlens: Tensor, *,
                     max_suffix_length: int = 32, scale: float = ROSA_SOFT_DEFAULT_SCALE,
                     dropout_p: float = ROSA_SOFT_DEFAULT_DROPOUT_P,
                     mismatch_scale: float = ROSA_SOFT_DEFAULT_MISMATCH_SCALE) -> Tensor:
    """Run RosaSoft independently over CUDA-packed variable-length sequences."""
    max_suffix_length = _validate_cuda_varlen_call(query, key, value, cu_seqlens,
                                                   max_suffix_length, scale, dropout_p,
                                                   mismatch_scale)
    needs_backward = torch.is_grad_enabled() and any(
        t.requires_grad for t in (query, key, value))
    if not needs_backward:
        return torch.ops.rosa_soft.hard_forward_varlen(query, key, value, cu_seqlens,
                                                       max_suffix_length)[0]
    dropout_seed = make_dropout_seed(query, dropout_p, needs_backward)
    return _HardForwardSoftVjpVarlenFunction.apply(query, key, value, cu_seqlens, dropout_seed,
                                                   max_suffix_length, float(scale),
                                                   float(dropout_p), float(mismatch_scale))
