"""rosa_soft_b200 -- sm_100a implementation of the rosa_soft operator family.

Drop-in for the operator surface of the reference package (``rosa_soft/__init__.py``:
exports :194-202, capability record :105-118, loader :20-30, registration checks :60-95):
``import rosa_soft_b200 as rosa_soft`` gives the same ``rosa_soft`` / ``rosa_soft_varlen``
callables, ``BUILD_CAPABILITIES`` and ``torch.ops.rosa_soft.*`` schemas.  The compiled
extension is mandatory: importing this package without it raises, and there is no CPU or
pure-PyTorch fallback behind the public operators.
"""
from __future__ import annotations

import importlib as _importlib
from dataclasses import dataclass as _dataclass

import torch as _torch

__version__ = "0.1.0"

_REQUIRED_CUDA_OPERATORS = (
    "hard_forward",
    "hard_forward_varlen",
    "surrogate_vjp_masked",
    "surrogate_vjp_varlen_masked",
)


def _load_compiled_extension():
    try:
        return _importlib.import_module(f"{__name__}._C")
    except ImportError as error:
        raise ImportError(
            "rosa_soft_b200._C is missing or failed to load; build it with "
            "`python rosa_soft_b200/build.py` (needs nvcc with sm_100a support). "
            "This package has no fallback implementation."
        ) from error


def _has_dispatch_kernel(operator: str, dispatch_key: str) -> bool:
    try:
        return bool(_torch._C._dispatch_has_kernel_for_dispatch_key(operator, dispatch_key))
    except RuntimeError:
        return False


_C = _load_compiled_extension()
_cuda_operator_flags = tuple(
    _has_dispatch_kernel(f"rosa_soft::{name}", "CUDA") for name in _REQUIRED_CUDA_OPERATORS
)
if not all(_cuda_operator_flags):
    raise RuntimeError(
        "rosa_soft_b200._C loaded with an incomplete CUDA operator registration; the "
        "extension is stale or incompatible with this package"
    )


@_dataclass(frozen=True, slots=True)
class BuildCapabilities:
    variant: str
    compiled_extension: bool
    rosa_runtime: bool
    rosa_soft_cuda: bool


BUILD_CAPABILITIES = BuildCapabilities(
    variant="cuda",
    compiled_extension=True,
    rosa_runtime=True,   # the GPU-resident streaming runtime of runtime.py
    rosa_soft_cuda=True,
)

from .inference import rosa_hard_inference  # noqa: E402
from .inspection import (HardRouteDiagnostics, HardRouteInspection, SymbolHealth,  # noqa: E402
                         inspect_hard_routes, summarize_hard_routes, symbol_health)
from .runtime import RosaRuntime  # noqa: E402
from .soft import rosa_soft, rosa_soft_varlen  # noqa: E402

__all__ = [
    "__version__",
    "BUILD_CAPABILITIES",
    "HardRouteInspection",
    "RosaRuntime",
    "inspect_hard_routes",
    "summarize_hard_routes",
    "symbol_health",
    "HardRouteDiagnostics",
    "SymbolHealth",
    "rosa_hard_inference",
    "rosa_soft",
    "rosa_soft_varlen",
]
