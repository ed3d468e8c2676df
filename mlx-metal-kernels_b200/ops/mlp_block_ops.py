"""Quantized linear / gate-up projection / full MLP block, CUDA backend.

Mirrors ops/mlp_block_ops.py of the reference.  Every per-stage backend string other than
``"reference"`` selects the CUDA kernels; when all four stages are on CUDA the block runs as two
launches: [residual add + RMSNorm + gate/up + SwiGLU] and [down projection + residual add].
"""
from __future__ import annotations

import math

import torch

from . import _cabi
from .activation_ops import fused_swiglu, swiglu
from .fused_ops import residual_add
from .quant_ops import (
    gate_up_rows,
    matvec_rows,
    q4_gate_up_matvec_tiled,
    q4_matvec_decode,
    q8_gate_up_matvec_tiled,
    q8_matvec_decode,
)


def _validate_bits(bits: int) -> int:
    if bits not in (4, 8):
        raise ValueError(f"bits must be 4 or 8, got {bits}")
    return bits


def _normalize_hidden_input(x):
    if x.ndim == 2:
        return x, tuple(x.shape)
    if x.ndim == 3:
        return x.reshape(x.shape[0] * x.shape[1], x.shape[2]), tuple(x.shape)
    raise ValueError(f"x must have shape [B,K], [B,1,K], or [B,S,K], got {tuple(x.shape)}")


def _restore_hidden_output(y2d, original_shape):
    if len(original_shape) == 2:
        return y2d
    return y2d.reshape(original_shape[:-1] + (y2d.shape[-1],))


def _validate_quantized_linear_shapes(x2d, w, scales, zeros, *, bits, group_size, name):
    _validate_bits(bits)
    if group_size <= 0:
        raise ValueError(f"group_size must be positive, got {group_size}")
    if x2d.ndim != 2:
        raise ValueError(f"{name} input must normalize to [rows,K], got {tuple(x2d.shape)}")
    if w.ndim != 2:
        raise ValueError(f"{name} weights must be 2-D, got {tuple(w.shape)}")
    in_dim = x2d.shape[1]
    out_dim = w.shape[0]
    if bits == 4:
        expected_cols = math.ceil(in_dim / 2)
        if w.shape[1] != expected_cols:
            raise ValueError(f"{name} q4 weights must have shape [{out_dim},{expected_cols}], got {tuple(w.shape)}")
    elif w.shape[1] != in_dim:
        raise ValueError(f"{name} q8 weights must have shape [{out_dim},{in_dim}], got {tuple(w.shape)}")
    groups = math.ceil(in_dim / group_size)
    if tuple(scales.shape) != (out_dim, groups):
        raise ValueError(f"{name} scales must have shape {(out_dim, groups)}, got {tuple(scales.shape)}")
    if zeros is not None and tuple(zeros.shape) != (out_dim, groups):
        raise ValueError(f"{name} zeros must have shape {(out_dim, groups)}, got {tuple(zeros.shape)}")
    return in_dim, out_dim


def quantized_linear(x, w, scales, zeros=None, *, bits=4, group_size=32, backend="auto"):
    """[B,K] / [B,S,K] -> same leading shape with N features (ops/mlp_block_ops.py:77-101)."""
    x2d, original_shape = _normalize_hidden_input(x)
    _validate_quantized_linear_shapes(x2d, w, scales, zeros, bits=bits, group_size=group_size, name="quantized_linear")
    if backend == "reference":
        _cabi.reference_unavailable("quantized_linear")
    fn = q4_matvec_decode if bits == 4 else q8_matvec_decode
    y2d = fn(x2d, w, scales, zeros, group_size=group_size, backend=backend)
    return _restore_hidden_output(y2d, original_shape)


def swiglu_down_project(gate, up, down_w, down_scales, down_zeros=None, *, bits=4, group_size=32,
                        activation_backend="metal", matvec_backend="metal_tiled"):
    """ops/mlp_block_ops.py:104-125."""
    if activation_backend == "reference":
        _cabi.reference_unavailable("swiglu_down_project")
    hidden = swiglu(gate, up, backend=activation_backend)
    return quantized_linear(hidden, down_w, down_scales, down_zeros, bits=bits, group_size=group_size,
                            backend=matvec_backend)


_GATE_UP_ERR = "backend must be one of 'reference', 'metal_tiled', 'metal_parallel', 'metal_gate_up_tiled', 'cuda'"


def quantized_gate_up_projection(x, gate_w, gate_scales, up_w, up_scales, *, gate_zeros=None, up_zeros=None, bits=4,
                                 group_size=32, backend="metal_tiled"):
    """(gate, up) = (Wg x, Wu x).  Note the argument order: weights and scales interleaved per
    projection (ops/mlp_block_ops.py:128-233)."""
    _validate_bits(bits)
    if backend not in {"reference", "metal_tiled", "metal_parallel", "metal_gate_up_tiled", "cuda"}:
        raise ValueError(_GATE_UP_ERR)
    if backend == "reference" or _cabi.safe_mode_enabled():
        _cabi.reference_unavailable("quantized_gate_up_projection")
    fn = q4_gate_up_matvec_tiled if bits == 4 else q8_gate_up_matvec_tiled
    return fn(x, gate_w, up_w, gate_scales, up_scales, gate_zeros, up_zeros, group_size=group_size)


def _resolve_mlp_backends(*, backend_preset=None, norm_backend="metal", matvec_backend="metal_tiled",
                          activation_backend="metal", residual_backend="metal"):
    """ops/mlp_block_ops.py:236-255, plus the preset ``"cuda"``."""
    if backend_preset is None:
        return norm_backend, matvec_backend, activation_backend, residual_backend
    mapping = {
        "reference": ("reference", "reference", "reference", "reference"),
        "metal": ("metal", "metal_tiled", "metal", "metal"),
        "parallel": ("metal", "metal_parallel", "metal", "metal"),
        "tiled": ("metal", "metal_tiled", "metal", "metal"),
        "fused_experimental": ("metal", "metal_gate_up_tiled", "metal_fused", "metal"),
        "cuda": ("cuda", "cuda", "cuda", "cuda"),
    }
    if backend_preset not in mapping:
        raise ValueError(f"backend_preset must be one of {tuple(mapping)}, got {backend_preset}")
    return mapping[backend_preset]


def reference_quantized_mlp_block(*args, **kwargs):
    _cabi.reference_unavailable("reference_quantized_mlp_block")


_STAGE_OK = {
    "norm": ("auto", "metal", "cuda"),
    "matvec": ("auto", "metal", "metal_tiled", "metal_parallel", "metal_gate_up_tiled", "cuda"),
    "activation": ("auto", "metal", "metal_fused", "cuda"),
    "residual": ("auto", "metal", "cuda"),
}


def quantized_mlp_block(x, residual, norm_weight, gate_w, gate_scales, up_w, up_scales, down_w, down_scales, *,
                        gate_zeros=None, up_zeros=None, down_zeros=None, bits=4, group_size=32, eps=1e-5,
                        backend_preset=None, norm_backend="metal", matvec_backend="metal_tiled",
                        activation_backend="metal", residual_backend="metal", return_intermediates=False):
    """z = x + residual; n = rmsnorm(z); g,u = Wg n, Wu n; m = silu(g)*u; d = Wd m; out = z + d, every
    stage rounded to x.dtype (ops/mlp_block_ops.py:301-364).  With ``return_intermediates`` also
    returns ``{"z","normed","gate","up","mlp","down"}``."""
    if x.shape != residual.shape:
        raise ValueError(f"x and residual must have identical shapes, got {tuple(x.shape)}, {tuple(residual.shape)}")
    if x.ndim != 3:
        raise ValueError(f"x and residual must have shape [B,S,D], got {tuple(x.shape)}")
    if tuple(norm_weight.shape) != (x.shape[-1],):
        raise ValueError(f"norm_weight must have shape {(x.shape[-1],)}, got {tuple(norm_weight.shape)}")
    stages = _resolve_mlp_backends(backend_preset=backend_preset, norm_backend=norm_backend,
                                   matvec_backend=matvec_backend, activation_backend=activation_backend,
                                   residual_backend=residual_backend)
    if "reference" in stages or _cabi.safe_mode_enabled():
        _cabi.reference_unavailable("quantized_mlp_block")
    for stage, value in zip(("norm", "matvec", "activation", "residual"), stages):
        if value not in _STAGE_OK[stage]:
            raise ValueError(f"{stage}_backend must be one of {('reference',) + _STAGE_OK[stage]}, got {value!r}")
    _validate_bits(bits)
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"x dtype must be float16 or bfloat16, got {x.dtype}")

    B, S, D = x.shape
    x2d = x.reshape(B * S, D)
    r2d = residual.reshape(B * S, D)
    _validate_quantized_linear_shapes(x2d, gate_w, gate_scales, gate_zeros, bits=bits, group_size=group_size,
                                      name="gate")
    _validate_quantized_linear_shapes(x2d, up_w, up_scales, up_zeros, bits=bits, group_size=group_size, name="up")
    inter = gate_w.shape[0]
    res = gate_up_rows(bits, x2d, gate_w, up_w, gate_scales, up_scales, gate_zeros, up_zeros, group_size,
                       want_gate_up=return_intermediates, want_act=True, residual_in=r2d, norm_weight=norm_weight,
                       eps=eps, want_z=True, want_normed=return_intermediates)
    mlp2d, z2d = res["act"], res["z"]
    _validate_quantized_linear_shapes(mlp2d, down_w, down_scales, down_zeros, bits=bits, group_size=group_size,
                                      name="down")
    if not return_intermediates:
        out2d = matvec_rows(bits, mlp2d, down_w, down_scales, down_zeros, group_size, residual=z2d)
        return out2d.reshape(B, S, -1)
    down2d = matvec_rows(bits, mlp2d, down_w, down_scales, down_zeros, group_size)
    out2d = residual_add(z2d, down2d)
    shape = lambda t, n: t.reshape(B, S, n)
    return shape(out2d, D), {
        "z": shape(z2d, D), "normed": shape(res["normed"], D), "gate": shape(res["gate"], inter),
        "up": shape(res["up"], inter), "mlp": shape(mlp2d, inter), "down": shape(down2d, D),
    }


def quantized_mlp_decode_step(x, norm_weight, gate_w, gate_scales, up_w, up_scales, down_w, down_scales, *,
                              gate_zeros=None, up_zeros=None, down_zeros=None, bits=4, group_size=32, eps=1e-5,
                              backend_preset="tiled"):
    """The reference passes ``residual = x`` here, so z = 2x (ops/mlp_block_ops.py:367-404)."""
    if backend_preset == "parallel":
        backend_preset = "tiled"
    return quantized_mlp_block(x, x, norm_weight, gate_w, gate_scales, up_w, up_scales, down_w, down_scales,
                               gate_zeros=gate_zeros, up_zeros=up_zeros, down_zeros=down_zeros, bits=bits,
                               group_size=group_size, eps=eps, backend_preset=backend_preset)


__all__ = [
    "quantized_linear", "swiglu_down_project", "quantized_gate_up_projection", "reference_quantized_mlp_block",
    "quantized_mlp_block", "quantized_mlp_decode_step", "fused_swiglu",
]
