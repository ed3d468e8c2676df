"""Oracle (test infrastructure): quantized linear and the quantized MLP block.

Restates the all-"reference" route through ops/mlp_block_ops.py:77-101,
128-166 and 301-364 of the reference.  Every stage result is rounded to the
activation dtype before the next stage uses it.
"""
from __future__ import annotations

import math

import torch

from .elementwise_ops import reference_residual_add, reference_rms_norm, reference_swiglu
from .quant_ops import reference_q4_matvec_decode, reference_q8_matvec_decode


def _validate_bits(bits):
    if bits not in (4, 8):
        raise ValueError(f"bits must be 4 or 8, got {bits}")


def reference_quantized_linear(x, w, scales, zeros=None, *, bits=4, group_size=32):
    """ops/mlp_block_ops.py:77-101 with backend="reference"."""
    if x.ndim == 2:
        x2d, shape = x, tuple(x.shape)
    elif x.ndim == 3:
        x2d, shape = x.reshape(x.shape[0] * x.shape[1], x.shape[2]), tuple(x.shape)
    else:
        raise ValueError(f"x must have shape [B,K], [B,1,K], or [B,S,K], got {tuple(x.shape)}")
    _validate_bits(bits)
    if group_size <= 0:
        raise ValueError(f"group_size must be positive, got {group_size}")
    if w.ndim != 2:
        raise ValueError(f"quantized_linear weights must be 2-D, got {tuple(w.shape)}")
    in_dim, out_dim = x2d.shape[1], w.shape[0]
    cols = math.ceil(in_dim / 2) if bits == 4 else in_dim
    if w.shape[1] != cols:
        raise ValueError(f"quantized_linear q{bits} weights must have shape [{out_dim},{cols}], got {tuple(w.shape)}")
    groups = math.ceil(in_dim / group_size)
    if tuple(scales.shape) != (out_dim, groups):
        raise ValueError(f"quantized_linear scales must have shape {(out_dim, groups)}, got {tuple(scales.shape)}")
    if zeros is not None and tuple(zeros.shape) != (out_dim, groups):
        raise ValueError(f"quantized_linear zeros must have shape {(out_dim, groups)}, got {tuple(zeros.shape)}")
    fn = reference_q4_matvec_decode if bits == 4 else reference_q8_matvec_decode
    y2d = fn(x2d, w, scales, zeros, group_size=group_size)
    if len(shape) == 2:
        return y2d
    return y2d.reshape(shape[:-1] + (y2d.shape[-1],))


def reference_quantized_mlp_block(x, residual, norm_weight, gate_w, gate_scales, up_w, up_scales,
                                  down_w, down_scales, *, gate_zeros=None, up_zeros=None, down_zeros=None,
                                  bits=4, group_size=32, eps=1e-5, return_intermediates=False):
    """z=x+res; n=rms(z); g,u=Wg n,Wu n; m=silu(g)*u; d=Wd m; out=z+d
    (ops/mlp_block_ops.py:258-298 -> 301-364)."""
    if x.shape != residual.shape:
        raise ValueError(f"x and residual must have identical shapes, got {tuple(x.shape)}, {tuple(residual.shape)}")
    if x.ndim != 3:
        raise ValueError(f"x and residual must have shape [B,S,D], got {tuple(x.shape)}")
    if tuple(norm_weight.shape) != (x.shape[-1],):
        raise ValueError(f"norm_weight must have shape {(x.shape[-1],)}, got {tuple(norm_weight.shape)}")
    z = reference_residual_add(x, residual)
    normed = reference_rms_norm(z, norm_weight, eps=eps)
    gate = reference_quantized_linear(normed, gate_w, gate_scales, gate_zeros, bits=bits, group_size=group_size)
    up = reference_quantized_linear(normed, up_w, up_scales, up_zeros, bits=bits, group_size=group_size)
    mlp = reference_swiglu(gate, up)
    down = reference_quantized_linear(mlp, down_w, down_scales, down_zeros, bits=bits, group_size=group_size)
    out = reference_residual_add(z, down)
    if not return_intermediates:
        return out
    return out, {"z": z, "normed": normed, "gate": gate, "up": up, "mlp": mlp, "down": down}
