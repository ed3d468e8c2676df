"""RMSNorm (reference ops/norm_ops.py:30-85): y = cast(x * rsqrt(mean(x^2) + eps) * w)."""
from __future__ import annotations

import torch

from . import _cabi

_FLOAT = (torch.float16, torch.bfloat16, torch.float32)


def _validate_inputs(x, weight):
    if x.ndim != 3:
        raise ValueError(f"x must be 3-D [B,S,D], got shape {tuple(x.shape)}")
    if weight.ndim != 1:
        raise ValueError(f"weight must be 1-D [D], got shape {tuple(weight.shape)}")
    B, S, D = x.shape
    if D != weight.shape[0]:
        raise ValueError(f"weight shape must be [D] with D={D}, got {tuple(weight.shape)}")
    if B <= 0 or S <= 0 or D <= 0:
        raise ValueError(f"Invalid x shape: {tuple(x.shape)}")
    if x.dtype not in _FLOAT:
        raise TypeError(f"x dtype must be float16, bfloat16, or float32, got {x.dtype}")
    if weight.dtype not in _FLOAT:
        raise TypeError(f"weight dtype must be float16, bfloat16, or float32, got {weight.dtype}")
    return B, S, D


def rmsnorm_rows(x2d, residual2d, weight, eps, want_z):
    """Shared launcher: rows [R,D] (fp16/bf16), optional residual, weight in its own dtype."""
    _cabi.require_cuda(x2d, residual2d, weight)
    x2d = _cabi.contiguous(x2d)
    residual2d = None if residual2d is None else _cabi.contiguous(residual2d.to(x2d.dtype))
    weight = _cabi.contiguous(weight)
    y = torch.empty_like(x2d)
    z = torch.empty_like(x2d) if want_z else None
    R, D = x2d.shape
    _cabi.check(
        _cabi.load().b200q_rmsnorm_residual(x2d.data_ptr(), _cabi.ptr(residual2d), weight.data_ptr(), y.data_ptr(),
                                            _cabi.ptr(z), R, D, float(eps), _cabi.dtype_code(x2d.dtype),
                                            _cabi.dtype_code(weight.dtype), _cabi.stream()),
        "b200q_rmsnorm_residual",
    )
    return y, z


def reference_rms_norm(x, weight, eps: float = 1e-5):
    _cabi.reference_unavailable("reference_rms_norm")


def rms_norm(x, weight, eps: float = 1e-5, *, backend: str = "auto"):
    B, S, D = _validate_inputs(x, weight)
    name = backend.lower()
    if _cabi.safe_mode_enabled() or name == "reference":
        _cabi.reference_unavailable("rms_norm")
    if name not in ("auto", "metal", "cuda"):
        raise ValueError("backend must be one of 'reference', 'metal', 'auto', 'cuda'")
    if x.dtype == torch.float32:
        raise TypeError("the CUDA backend normalises float16 or bfloat16 rows")
    y, _ = rmsnorm_rows(x.reshape(B * S, D), None, weight, eps, False)
    return y.reshape(B, S, D)
