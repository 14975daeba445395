"""Routing inspection on the GPU, outside the training API.

The reference's ``inspect_rosa_soft`` (rosa_soft/testing.py:49-117) materialises
``[B, H, T, T + 1]`` tensors of suffix lengths, soft scores and route probabilities with
PyTorch operations, which limits it to short sequences.  The part of it that diagnostics read at
scale -- which route every position selected and how long the winning match was
(``selected_route_indices``, the selected entry of ``exact_suffix_lengths``; consumers in
rosa_soft/diagnostics.py:210-360) -- is a by-product of the hard forward kernel here and costs
no extra matching pass.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import cabi
from . import soft_contract as _contract


@dataclass(frozen=True)
class HardRouteInspection:
    selected_route_indices: Tensor    # int64 [B, H, T] (dense) or [H, N] (packed); 0 = null route
    selected_match_lengths: Tensor    # int64, same shape; 0 for the null route
    effective_max_suffix_length: int

    @property
    def null_route_fraction(self) -> float:
        return float((self.selected_route_indices == 0).float().mean())

    @property
    def mean_match_length(self) -> float:
        hit = self.selected_route_indices > 0
        return float(self.selected_match_lengths[hit].float().mean()) if bool(hit.any()) else 0.0


@torch.no_grad()
def inspect_hard_routes(query: Tensor, key: Tensor, value: Tensor,
                        cu_seqlens: Optional[Tensor] = None, *,
                        max_suffix_length: int = 32) -> Tuple[Tensor, HardRouteInspection]:
    """Hard output plus the routing decision behind it.

    Dense ``[B, T, H, D]`` inputs, or packed ``[N, H, D]`` with ``cu_seqlens``.  Route indices
    follow the reference's convention: route ``a`` in ``[1, i]`` reads ``value[a]`` and ends its
    match at key ``a - 1``; 0 is the null route.  Layout ``[B, H, T]`` as in the reference.
    """
    if not query.is_cuda:
        raise ValueError("inspect_hard_routes requires CUDA tensors")
    dense = cu_seqlens is None
    if dense:
        horizon = _contract.validate_rosa_soft_inputs(query, key, value, max_suffix_length, 1.0, 0.0,
                                                     3.0)
        B, T, H, D = query.shape
        flat = lambda t: t.contiguous().reshape(B * T, *t.shape[2:])
        seqs = (B, T)
    else:
        horizon = _contract.validate_rosa_soft_varlen_inputs(query, key, value, cu_seqlens,
                                                             max_suffix_length, 1.0, 0.0, 3.0)
        H = query.shape[1]
        flat = lambda t: t.contiguous()
        seqs = cu_seqlens.to(torch.int32)
    q, k, v = flat(query), flat(key), flat(value)
    out, _, _, _, ws = cabi.hard_forward(q, k, v, seqs, horizon, want_routes=False)
    N = q.shape[0]
    num_seq = seqs[0] if dense else seqs.numel() - 1
    route, length = cabi.hard_forward_routes(ws, N, H, num_seq)
    if dense:
        out = out.reshape(B, T, H, -1)
        to_layout = lambda t: t.reshape(B, T, H).permute(0, 2, 1).to(torch.int64).contiguous()
    else:
        to_layout = lambda t: t.t().to(torch.int64).contiguous()
    return out, HardRouteInspection(to_layout(route), to_layout(length), horizon)
