"""Residual add and RMSNorm+residual (reference ops/fused_ops.py:149-241)."""
from __future__ import annotations

import torch

from . import _cabi
from .norm_ops import rmsnorm_rows

_ACT = (torch.float16, torch.bfloat16)


def reference_residual_add(x, residual):
    _cabi.reference_unavailable("reference_residual_add")


def residual_add(x, residual, *, backend: str = "auto"):
    """out = cast(float(x) + float(residual))."""
    if x.shape != residual.shape:
        raise ValueError(f"x and residual must have identical shapes, got {tuple(x.shape)}, {tuple(residual.shape)}")
    if x.dtype not in _ACT:
        raise TypeError(f"x dtype must be float16 or bfloat16, got {x.dtype}")
    name = backend.lower()
    if _cabi.safe_mode_enabled() or name == "reference":
        _cabi.reference_unavailable("residual_add")
    if name not in ("auto", "metal", "cuda"):
        raise ValueError("backend must be one of 'reference', 'metal', 'auto', 'cuda'")
    _cabi.require_cuda(x, residual)
    x = _cabi.contiguous(x)
    residual = _cabi.contiguous(residual.to(x.dtype))
    out = torch.empty_like(x)
    _cabi.check(
        _cabi.load().b200q_residual_add(x.data_ptr(), residual.data_ptr(), out.data_ptr(), x.numel(),
                                        _cabi.dtype_code(x.dtype), _cabi.stream()),
        "b200q_residual_add",
    )
    return out


def reference_rmsnorm_residual(x, residual, weight, eps: float = 1e-5, *, return_residual: bool = False):
    _cabi.reference_unavailable("reference_rmsnorm_residual")


def rmsnorm_residual(x, residual, weight, eps: float = 1e-5, *, return_residual: bool = False, backend: str = "auto"):
    """z = cast(x + residual); y = rmsnorm(z); returns y or (y, z)."""
    if x.shape != residual.shape:
        raise ValueError(f"x and residual must have identical shapes, got {tuple(x.shape)}, {tuple(residual.shape)}")
    if weight.ndim != 1 or x.shape[-1] != weight.shape[0]:
        raise ValueError(f"weight must have shape [D] with D={x.shape[-1]}, got {tuple(weight.shape)}")
    if x.dtype not in _ACT:
        raise TypeError(f"x dtype must be float16 or bfloat16, got {x.dtype}")
    name = backend.lower()
    if _cabi.safe_mode_enabled() or name == "reference":
        _cabi.reference_unavailable("rmsnorm_residual")
    if name not in ("auto", "metal", "cuda"):
        raise ValueError("backend must be one of 'reference', 'metal', 'auto', 'cuda'")
    D = x.shape[-1]
    y, z = rmsnorm_rows(x.reshape(-1, D), residual.reshape(-1, D), weight, eps, True)
    y = y.reshape(x.shape)
    return (y, z.reshape(x.shape)) if return_residual else y
