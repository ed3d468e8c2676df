"""SwiGLU (reference ops/activation_ops.py:83-153): out = cast(silu(gate) * up)."""
from __future__ import annotations

import torch

from . import _cabi

_ACT = (torch.float16, torch.bfloat16)


def _validate(gate, up, name_ndim=None):
    if gate.shape != up.shape:
        raise ValueError(f"gate and up must have identical shapes, got {tuple(gate.shape)}, {tuple(up.shape)}")
    if gate.dtype not in _ACT:
        raise TypeError(f"gate dtype must be float16 or bfloat16, got {gate.dtype}")
    if up.dtype not in _ACT:
        raise TypeError(f"up dtype must be float16 or bfloat16, got {up.dtype}")


def _launch(gate, up):
    _cabi.require_cuda(gate, up)
    gate = _cabi.contiguous(gate)
    up = _cabi.contiguous(up.to(gate.dtype))
    out = torch.empty_like(gate)
    dim = gate.shape[-1]
    rows = gate.numel() // dim
    _cabi.check(
        _cabi.load().b200q_swiglu(gate.data_ptr(), up.data_ptr(), out.data_ptr(), rows, dim,
                                  _cabi.dtype_code(gate.dtype), _cabi.stream()),
        "b200q_swiglu",
    )
    return out


def reference_swiglu(gate, up):
    _cabi.reference_unavailable("reference_swiglu")


def swiglu(gate, up, *, backend: str = "auto"):
    """[B,S,D] inputs (ops/activation_ops.py:91-115)."""
    if gate.ndim != 3:
        raise ValueError(f"gate and up must be 3-D [B,S,D], got {tuple(gate.shape)}, {tuple(up.shape)}")
    _validate(gate, up)
    name = backend.lower()
    if _cabi.safe_mode_enabled() or name == "reference":
        _cabi.reference_unavailable("swiglu")
    if name not in ("auto", "metal", "cuda"):
        raise ValueError("backend must be one of 'reference', 'metal', 'auto', 'cuda'")
    return _launch(gate, up)


def fused_swiglu(gate, up, *, backend: str = "metal_fused"):
    """[rows,D] or [B,S,D] inputs (ops/activation_ops.py:118-153)."""
    if gate.ndim not in (2, 3) or gate.shape != up.shape:
        raise ValueError(f"gate and up must have shape [rows,D] or [B,S,D], got {tuple(gate.shape)}, {tuple(up.shape)}")
    _validate(gate, up)
    name = backend.lower()
    if _cabi.safe_mode_enabled() or name == "reference":
        _cabi.reference_unavailable("fused_swiglu")
    if name == "metal" and gate.ndim != 3:
        raise ValueError("backend='metal' for fused_swiglu requires [B,S,D] inputs; use 'metal_fused' for flattened shapes")
    if name not in ("auto", "metal", "metal_fused", "cuda"):
        raise ValueError("backend must be one of 'reference', 'metal', 'metal_fused', 'auto', 'cuda'")
    return _launch(gate, up)
