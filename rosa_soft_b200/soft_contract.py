"""Host-side contract of the rosa_soft operator family.

Names, defaults, argument meaning, return values and error texts are those of the
reference's ``rosa_soft/soft_contract.py`` (defaults :12-15, dropout seed :18-31, control
validation :34-66, dense inputs :69-129, packed inputs :132-208, float32 scalar ranges
:211-248), because callers and tests match on them.  The checks are written as ordered rule
tables: the first rule that fails raises, which reproduces the reference's error precedence.
Nothing here touches tensor data except the value check of a CPU ``cu_seqlens``; CUDA offsets
are validated on the device by the operator.
"""
from __future__ import annotations

import math
import operator
from typing import Callable, Iterable, Tuple

import torch
from torch import Tensor

ROSA_SOFT_DEFAULT_SCALE = 1.0
ROSA_SOFT_DEFAULT_DROPOUT_P = 0.0
ROSA_SOFT_DEFAULT_MISMATCH_SCALE = 3.0
ROSA_SOFT_NULL_ROUTE_SCORE = 0.5

_MAX_DROPOUT_P = 1.0 - 2.0 ** -24
_Rule = Tuple[Callable[[], bool], str]


def _enforce(rules: Iterable[_Rule]) -> None:
    """Raise ``ValueError(message)`` for the first rule whose predicate is false."""
    for holds, message in rules:
        if not holds():
            raise ValueError(message)


def make_dropout_seed(reference: Tensor, dropout_p: float, needs_backward: bool) -> Tensor:
    """int64 scalar drawn from ``reference.device``'s generator iff a backward with dropout
    will run; an empty int64 tensor otherwise (no random number is consumed then).  Drawing on
    the device is what lets ``torch.cuda.manual_seed`` / ``preserve_rng_state`` replay masks."""
    wanted = needs_backward and float(dropout_p) != 0.0
    if wanted:
        return torch.randint(0, torch.iinfo(torch.int64).max, (), dtype=torch.int64,
                             device=reference.device)
    return torch.empty(0, dtype=torch.int64, device=reference.device)


def _is_plain_finite(value) -> bool:
    return not isinstance(value, bool) and math.isfinite(float(value))


def _validate_static_controls(max_suffix_length, scale, dropout_p, mismatch_scale,
                              sequence_length_bound: int) -> int:
    try:
        if isinstance(max_suffix_length, bool):
            raise TypeError
        horizon = operator.index(max_suffix_length)
    except TypeError:
        raise TypeError("max_suffix_length must be an integer") from None
    _enforce((
        (lambda: horizon >= 1, "max_suffix_length must be >= 1"),
        (lambda: _is_plain_finite(scale) and float(scale) > 0.0, "scale must be finite and > 0"),
        (lambda: _is_plain_finite(dropout_p) and 0.0 <= float(dropout_p) <= _MAX_DROPOUT_P,
         "dropout_p must be finite and in [0, 1 - 2^-24]"),
        (lambda: _is_plain_finite(mismatch_scale) and float(mismatch_scale) > 0.0,
         "mismatch_scale must be finite and > 0"),
    ))
    return min(horizon, sequence_length_bound)


def validate_rosa_soft_inputs(query: Tensor, key: Tensor, value: Tensor, max_suffix_length,
                              scale, dropout_p, mismatch_scale) -> int:
    """Dense ``(B, T, H, D)`` / ``(B, T, Hv, Dv)`` inputs; returns ``min(W, T)``."""
    q, k, v = query, key, value
    _enforce((
        (lambda: q.ndim == 4 and k.ndim == 4 and v.ndim == 4,
         "query, key, and value must have shape (B, T, H, D)"),
        (lambda: q.shape[:2] == k.shape[:2] and q.shape[:2] == v.shape[:2],
         "all inputs must share batch and sequence dimensions"),
        (lambda: q.size(2) == k.size(2), "query and key head counts must match"),
        (lambda: q.size(2) >= 1 and v.size(2) >= 1,
         "query and value must have at least one head"),
        (lambda: q.size(2) % v.size(2) == 0, "query heads must be divisible by value heads"),
        (lambda: q.size(3) == k.size(3), "query and key symbol dimensions must match"),
        (lambda: q.size(0) >= 1 and q.size(1) >= 1 and v.size(3) >= 1,
         "batch, sequence, and value dimensions must be >= 1"),
        (lambda: 1 <= q.size(3) <= 32, "query/key symbol dimension must be in [1, 32]"),
        (lambda: q.device == k.device == v.device, "all inputs must be on the same device"),
        (lambda: q.dtype == k.dtype == v.dtype, "all inputs must have the same dtype"),
        (lambda: q.is_floating_point() and k.is_floating_point() and v.is_floating_point(),
         "all inputs must be floating-point tensors"),
    ))
    return _validate_static_controls(max_suffix_length, scale, dropout_p, mismatch_scale, q.size(1))


def _offsets_rules(cu_seqlens: Tensor, tokens: int) -> Tuple[_Rule, ...]:
    offsets = cu_seqlens.tolist()
    return (
        (lambda: offsets[0] == 0, "cu_seqlens must start at zero"),
        (lambda: offsets[-1] == tokens, "cu_seqlens must end at the packed token count"),
        (lambda: all(a <= b for a, b in zip(offsets, offsets[1:])),
         "cu_seqlens must be nondecreasing"),
    )


def validate_rosa_soft_varlen_inputs(query: Tensor, key: Tensor, value: Tensor, cu_seqlens: Tensor,
                                     max_suffix_length, scale, dropout_p, mismatch_scale) -> int:
    """Packed ``(N, H, D)`` / ``(N, Hv, Dv)`` inputs with int32 offsets; returns ``min(W, N)``."""
    q, k, v, cu = query, key, value, cu_seqlens
    _enforce((
        (lambda: q.ndim == 3 and k.ndim == 3 and v.ndim == 3,
         "query, key, and value must have shape (N, H, D)"),
        (lambda: q.size(0) == k.size(0) == v.size(0),
         "all inputs must share the packed token dimension"),
        (lambda: q.size(0) >= 1, "packed token dimension must be >= 1"),
        (lambda: q.size(2) == k.size(2), "query and key symbol dimensions must match"),
        (lambda: q.size(1) == k.size(1), "query and key head counts must match"),
        (lambda: q.size(1) >= 1 and v.size(1) >= 1,
         "query and value must have at least one head"),
        (lambda: q.size(1) % v.size(1) == 0, "query heads must be divisible by value heads"),
        (lambda: 1 <= q.size(2) <= 32, "query/key symbol dimension must be in [1, 32]"),
        (lambda: v.size(2) >= 1, "value dimension must be >= 1"),
        (lambda: q.device == k.device == v.device == cu.device,
         "all inputs and cu_seqlens must be on the same device"),
        (lambda: q.dtype == k.dtype == v.dtype,
         "all floating-point inputs must have the same dtype"),
        (lambda: q.is_floating_point() and k.is_floating_point() and v.is_floating_point(),
         "query, key, and value must be floating-point tensors"),
        (lambda: cu.ndim == 1 and cu.numel() >= 2,
         "cu_seqlens must be a one-dimensional int32 tensor"),
        (lambda: cu.dtype == torch.int32, "cu_seqlens must have dtype int32"),
    ))
    if not cu.is_cuda:   # device offsets are checked by the operator, without a host sync
        _enforce(_offsets_rules(cu, q.size(0)))
    return _validate_static_controls(max_suffix_length, scale, dropout_p, mismatch_scale, q.size(0))


def validate_fp32_surrogate_scalars(max_suffix_length: int, scale, dropout_p, mismatch_scale) -> None:
    """The kernels take these controls as float32: each, and the products formed from them,
    must be representable."""
    lo, hi = torch.finfo(torch.float32).tiny, torch.finfo(torch.float32).max
    scale, dropout_p, mismatch_scale = float(scale), float(dropout_p), float(mismatch_scale)
    horizon = float(max_suffix_length)
    inverse_keep = 1.0 / (1.0 - dropout_p)
    _enforce((
        (lambda: math.isfinite(scale) and lo <= scale <= hi,
         "scale must be representable as a positive normal float32 value"),
        (lambda: scale <= hi / horizon, "max_suffix_length * scale must fit in float32"),
        (lambda: math.isfinite(inverse_keep) and inverse_keep <= hi,
         "1 / (1 - dropout_p) must fit in float32"),
        (lambda: lo <= mismatch_scale <= hi,
         "mismatch_scale must be representable as a positive normal float32 value"),
        (lambda: mismatch_scale <= hi / (horizon * scale),
         "mismatch_scale * max_suffix_length * scale must fit in float32"),
    ))
