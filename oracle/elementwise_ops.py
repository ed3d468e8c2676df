"""Oracle (test infrastructure): SwiGLU, RMSNorm, residual add.

fp32 math, one cast to the input dtype at the end of each function, exactly
where the reference casts.
"""
from __future__ import annotations

import torch


def reference_swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up with silu(g) = g / (1 + exp(-g))  (ops/activation_ops.py:83-88)."""
    if gate.shape != up.shape:
        raise ValueError(f"gate and up must have identical shapes, got {tuple(gate.shape)}, {tuple(up.shape)}")
    g = gate.to(torch.float32)
    u = up.to(torch.float32)
    silu = g / (1.0 + torch.exp(-g))
    return (silu * u).to(gate.dtype)


def reference_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w  (ops/norm_ops.py:47-52)."""
    if x.ndim != 3:
        raise ValueError(f"x must be 3-D [B,S,D], got shape {tuple(x.shape)}")
    if weight.ndim != 1:
        raise ValueError(f"weight must be 1-D [D], got shape {tuple(weight.shape)}")
    D = x.shape[-1]
    if D != weight.shape[0]:
        raise ValueError(f"weight shape must be [D] with D={D}, got {tuple(weight.shape)}")
    xf = x.to(torch.float32)
    variance = xf.square().mean(dim=-1, keepdim=True)
    inv_rms = torch.rsqrt(variance + float(eps))
    out = xf * inv_rms * weight.to(torch.float32).reshape(1, 1, D)
    return out.to(x.dtype)


def reference_residual_add(x: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """ops/fused_ops.py:149-152."""
    if x.shape != residual.shape:
        raise ValueError(f"x and residual must have identical shapes, got {tuple(x.shape)}, {tuple(residual.shape)}")
    return (x.to(torch.float32) + residual.to(torch.float32)).to(x.dtype)


def reference_rmsnorm_residual(x, residual, weight, eps: float = 1e-5, *, return_residual: bool = False):
    """z = x + residual (rounded), y = rmsnorm(z)  (ops/fused_ops.py:194-209)."""
    if x.shape != residual.shape:
        raise ValueError(f"x and residual must have identical shapes, got {tuple(x.shape)}, {tuple(residual.shape)}")
    if weight.ndim != 1 or x.shape[-1] != weight.shape[0]:
        raise ValueError(f"weight must have shape [D] with D={x.shape[-1]}, got {tuple(weight.shape)}")
    z = reference_residual_add(x, residual)
    zf = z.to(torch.float32)
    variance = zf.square().mean(dim=-1, keepdim=True)
    y = (zf * torch.rsqrt(variance + float(eps)) * weight.to(torch.float32)).to(x.dtype)
    return (y, z) if return_residual else y
