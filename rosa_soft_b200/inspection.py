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
    row_positions: Optional[Tensor] = None   # int64 [T] or [N]: position inside the sequence

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
    if dense:
        rows = torch.arange(T, device=query.device, dtype=torch.int64)
    else:
        # position of every packed token inside its own sequence
        starts = seqs.to(torch.int64)
        owner = torch.searchsorted(starts[1:].contiguous(), torch.arange(N, device=query.device),
                                   right=True)
        rows = torch.arange(N, device=query.device, dtype=torch.int64) - starts[owner]
    return out, HardRouteInspection(to_layout(route), to_layout(length), horizon, rows)


@dataclass(frozen=True)
class SymbolHealth:
    """The input-side figures of the reference's summary (rosa_soft/diagnostics.py:186-207)."""
    positive_fraction: float          # share of components with x > 0
    bit_imbalance: float              # mean over bits of 2 |P(x_d > 0) - 1/2|
    sign_margin_mean: float           # mean |x|
    sign_margin_low_quantile: float   # low quantile of |x|
    softsign_derivative_mean: float   # mean 1 / (1 + |x|)^2


@dataclass(frozen=True)
class HardRouteDiagnostics:
    """The figures of the reference's ``summarize_rosa_soft`` (rosa_soft/diagnostics.py:210-360)
    that follow from the hard routing decision and the inputs alone; the ones that need the
    quadratic route-probability tensor are not offered."""
    hard_nonnull_route_fraction: float
    hard_route_lag_mean: float               # mean of (row - route) over non-null rows; NaN if none
    selected_match_length_mean: float        # NaN if every row is null
    horizon_hit_fraction: float              # non-null rows whose match fills the horizon
    query: SymbolHealth
    key: SymbolHealth


def _quantile(values: Tensor, q: float) -> float:
    """Low quantile by linear interpolation of the order statistics (torch.quantile's default),
    on tensors of any size."""
    flat = values.reshape(-1).float()
    n = flat.numel()
    pos = q * (n - 1)
    lo = int(pos)
    hi = min(lo + 1, n - 1)
    a = float(torch.kthvalue(flat, lo + 1).values)
    b = float(torch.kthvalue(flat, hi + 1).values)
    return a + (b - a) * (pos - lo)


@torch.no_grad()
def symbol_health(logits: Tensor, low_quantile: float = 0.05) -> SymbolHealth:
    """Sign statistics of a ``[..., D]`` logit tensor (the Q or K input of the operator)."""
    if not 0.0 <= float(low_quantile) <= 1.0:
        raise ValueError("quantile must be in [0, 1]")
    x = logits.float()
    positive = (x > 0).float()
    per_bit = positive.reshape(-1, x.shape[-1]).mean(dim=0)
    margins = x.abs()
    return SymbolHealth(
        positive_fraction=float(positive.mean()),
        bit_imbalance=float((2.0 * (per_bit - 0.5).abs()).mean()),
        sign_margin_mean=float(margins.mean()),
        sign_margin_low_quantile=_quantile(margins, float(low_quantile)),
        softsign_derivative_mean=float((1.0 + margins).square().reciprocal().mean()))


@torch.no_grad()
def summarize_hard_routes(inspection: HardRouteInspection, query: Tensor, key: Tensor,
                          low_quantile: float = 0.05) -> HardRouteDiagnostics:
    """Route statistics from a :class:`HardRouteInspection` and the logits it was made from,
    computed with device-side reductions (a handful of scalars reach the host)."""
    routes, lengths = inspection.selected_route_indices, inspection.selected_match_lengths
    nonnull = routes > 0
    count = int(nonnull.sum())
    nan = float("nan")
    rows = inspection.row_positions
    if rows is None:
        raise ValueError("the inspection carries no row positions")
    lag = (rows.to(routes.device) - routes)[nonnull] if count else None
    return HardRouteDiagnostics(
        hard_nonnull_route_fraction=float(nonnull.float().mean()),
        hard_route_lag_mean=float(lag.float().mean()) if count else nan,
        selected_match_length_mean=float(lengths[nonnull].float().mean()) if count else nan,
        horizon_hit_fraction=(float((lengths[nonnull] >= inspection.effective_max_suffix_length)
                                    .float().mean()) if count else nan),
        query=symbol_health(query, low_quantile), key=symbol_health(key, low_quantile))
