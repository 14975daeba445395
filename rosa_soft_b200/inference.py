"""Batched hard inference on the GPU.

One call resolves whole streams: for every position and head the latest among the longest
suffix matches of the query history inside the key history (bounded by
``max_suffix_length``), exactly what feeding the same streams to the reference's CPU
``RosaRuntime`` returns (rosa_soft/csrc/rosa_runtime.cpp:41-45 match-then-extend, :120-131
capped query length, :455-467 successor payload; Python surface rosa_soft/runtime.py:605-651).
Symbols are integer words of up to 32 bits instead of the runtime's 8.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor


def rosa_hard_inference(query_symbols: Tensor, key_symbols: Tensor, payload: Tensor,
                        cu_seqlens: Optional[Tensor] = None, *,
                        max_suffix_length: int = 32) -> Tuple[Tensor, Tensor]:
    """Return ``(output, matched_key_end_positions)``.

    Dense form: symbols ``[streams, T, H]`` int32, payload ``[streams, T, Hp, Dp]`` float32.
    Packed form: symbols ``[N, H]``, payload ``[N, Hp, Dp]`` and int32 ``cu_seqlens``.
    ``matched_key_end_positions`` is int64, local to the stream, ``-1`` for no match;
    ``output`` is the payload row that follows the match (zeros for no match).
    """
    if isinstance(max_suffix_length, bool) or int(max_suffix_length) < 1:
        raise ValueError("max_suffix_length must be an integer >= 1")
    if not query_symbols.is_cuda:
        raise ValueError("rosa_hard_inference requires CUDA tensors")
    if query_symbols.dtype != torch.int32 or key_symbols.dtype != torch.int32:
        raise ValueError("symbols must be int32 words (bit patterns of up to 32 bits)")
    if payload.dtype != torch.float32:
        raise ValueError("payload must be float32")
    return torch.ops.rosa_soft.hard_inference(query_symbols, key_symbols, payload, cu_seqlens,
                                              int(max_suffix_length))
