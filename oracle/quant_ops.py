"""Oracle (test infrastructure): q4/q8 group-wise pack / dequant / matvec.

Restates ops/quant_ops.py of the reference on torch-CPU tensors.  Every cast
below sits where the reference has an ``astype``; nothing is fused.
"""
from __future__ import annotations

import math

import torch

_FLOAT_OUT = (torch.float16, torch.bfloat16)


def _normalize_out_dtype(out_dtype):
    # ops/quant_ops.py:147-152
    if out_dtype is None:
        return torch.float16
    if out_dtype not in _FLOAT_OUT:
        raise TypeError(f"out_dtype must be float16 or bfloat16, got {out_dtype}")
    return out_dtype


def _validate_group_params(M, K, scales, zeros, group_size):
    # ops/quant_ops.py:155-163
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    groups = math.ceil(K / group_size)
    if tuple(scales.shape) != (M, groups):
        raise ValueError(f"scales must have shape {(M, groups)}, got {tuple(scales.shape)}")
    if zeros is not None and tuple(zeros.shape) != (M, groups):
        raise ValueError(f"zeros must have shape {(M, groups)}, got {tuple(zeros.shape)}")
    return groups


def pack_q4(q_unpacked: torch.Tensor) -> torch.Tensor:
    """[M,K] codes -> [M,ceil(K/2)] bytes, low nibble = even k (ops/quant_ops.py:166-176)."""
    if q_unpacked.ndim != 2:
        raise ValueError(f"q_unpacked must be 2-D [M,K], got {tuple(q_unpacked.shape)}")
    q_int = q_unpacked.to(torch.uint8)
    if q_int.shape[1] % 2 != 0:
        pad = torch.zeros((q_int.shape[0], 1), dtype=torch.uint8)
        q_int = torch.cat([q_int, pad], dim=1)
    low = q_int[:, 0::2]
    high = q_int[:, 1::2]
    return (low + (high << 4)).to(torch.uint8)


def unpack_q4_reference(packed: torch.Tensor, K: int | None = None) -> torch.Tensor:
    """ops/quant_ops.py:179-188."""
    if packed.ndim != 2:
        raise ValueError(f"packed must be 2-D [M,K_packed], got {tuple(packed.shape)}")
    packed_u8 = packed.to(torch.uint8)
    low = packed_u8 & 0x0F
    high = (packed_u8 >> 4) & 0x0F
    unpacked = torch.stack([low, high], dim=-1).reshape(packed.shape[0], packed.shape[1] * 2)
    if K is not None:
        unpacked = unpacked[:, :K]
    return unpacked.to(torch.uint8)


def _expand(groupwise: torch.Tensor, group_size: int, K: int) -> torch.Tensor:
    return groupwise.to(torch.float32).repeat_interleave(group_size, dim=1)[:, :K]


def _dequant_codes(q_f32, scales, zeros, group_size, K, out_dtype):
    # ops/quant_ops.py:205-212 / 269-276: two separately rounded fp32 operations, then one cast.
    scale_full = _expand(scales, group_size, K)
    if zeros is None:
        out = q_f32 * scale_full
    else:
        zero_full = _expand(zeros, group_size, K)
        out = (q_f32 - zero_full) * scale_full
    return out.to(out_dtype)


def reference_dequant_q4(packed, scales, zeros=None, *, group_size: int = 32, out_dtype=None):
    """ops/quant_ops.py:191-212."""
    if packed.ndim != 2:
        raise ValueError(f"packed must be 2-D [M,K_packed], got {tuple(packed.shape)}")
    out_dtype = _normalize_out_dtype(out_dtype)
    M, K_packed = packed.shape
    K = K_packed * 2
    _validate_group_params(M, K, scales, zeros, group_size)
    q = unpack_q4_reference(packed, K=K).to(torch.float32)
    return _dequant_codes(q, scales, zeros, group_size, K, out_dtype)


def reference_dequant_q8(q, scales, zeros=None, *, group_size: int = 32, out_dtype=None):
    """ops/quant_ops.py:256-276."""
    if q.ndim != 2:
        raise ValueError(f"q must be 2-D [M,K], got {tuple(q.shape)}")
    out_dtype = _normalize_out_dtype(out_dtype)
    M, K = q.shape
    _validate_group_params(M, K, scales, zeros, group_size)
    return _dequant_codes(q.to(torch.float32), scales, zeros, group_size, K, out_dtype)


def reference_groupwise_dequant(q, scales, zeros=None, *, bits, group_size: int = 32, out_dtype=None):
    """ops/quant_ops.py:319-333 with backend="reference"."""
    if bits == 4:
        return reference_dequant_q4(q, scales, zeros, group_size=group_size, out_dtype=out_dtype)
    if bits == 8:
        return reference_dequant_q8(q, scales, zeros, group_size=group_size, out_dtype=out_dtype)
    raise ValueError(f"bits must be 4 or 8, got {bits}")


def _normalize_x_2d(x):
    # ops/quant_ops.py:336-342
    if x.ndim == 2:
        return x, x.shape[0], x.shape[1]
    if x.ndim == 3 and x.shape[1] == 1:
        squeezed = x[:, 0, :]
        return squeezed, squeezed.shape[0], squeezed.shape[1]
    raise ValueError(f"x must have shape [B,K] or [B,1,K], got {tuple(x.shape)}")


def _matmul_clip_cast(x2d, W):
    # ops/quant_ops.py:524-526: fp32 matmul of the dtype-rounded weights, clip to finfo, cast.
    result = x2d.to(torch.float32) @ W.to(torch.float32).T
    finfo = torch.finfo(x2d.dtype)
    return result.clamp(finfo.min, finfo.max).to(x2d.dtype)


def reference_q4_matvec_decode(x, packed_w, scales, zeros=None, *, group_size: int = 32):
    """ops/quant_ops.py:509-526.  Output is [B,N] even for a [B,1,K] input."""
    x2d, _, K = _normalize_x_2d(x)
    if packed_w.ndim != 2:
        raise ValueError(f"packed_w must be 2-D [N,K_packed], got {tuple(packed_w.shape)}")
    _, K_packed = packed_w.shape
    if K_packed * 2 != K:
        raise ValueError(f"packed_w implies K={K_packed * 2}, but x has K={K}")
    W = reference_dequant_q4(packed_w, scales, zeros, group_size=group_size, out_dtype=x2d.dtype)
    return _matmul_clip_cast(x2d, W)


def reference_q8_matvec_decode(x, q_w, scales, zeros=None, *, group_size: int = 32):
    """ops/quant_ops.py:574-588."""
    x2d, _, K = _normalize_x_2d(x)
    if q_w.ndim != 2 or q_w.shape[1] != K:
        raise ValueError(f"q_w must have shape [N,{K}], got {tuple(q_w.shape)}")
    W = reference_dequant_q8(q_w, scales, zeros, group_size=group_size, out_dtype=x2d.dtype)
    return _matmul_clip_cast(x2d, W)


def _normalize_hidden_rows_input(x):
    # ops/quant_ops.py:350-356
    if x.ndim == 2:
        return x, tuple(x.shape)
    if x.ndim == 3:
        return x.reshape(x.shape[0] * x.shape[1], x.shape[2]), tuple(x.shape)
    raise ValueError(f"x must have shape [rows,K] or [B,S,K], got {tuple(x.shape)}")


def reference_gate_up_matvec(x, gate_w, up_w, gate_scales, up_scales, gate_zeros=None, up_zeros=None,
                             *, bits: int, group_size: int = 32):
    """What q4/q8_gate_up_matvec_tiled (ops/quant_ops.py:634-738) must equal: the two
    reference matvecs of the same rows, reshaped like ops/quant_ops.py:359-362."""
    x2d, shape = _normalize_hidden_rows_input(x)
    fn = reference_q4_matvec_decode if bits == 4 else reference_q8_matvec_decode
    gate = fn(x2d, gate_w, gate_scales, gate_zeros, group_size=group_size)
    up = fn(x2d, up_w, up_scales, up_zeros, group_size=group_size)
    if len(shape) == 3:
        gate = gate.reshape(shape[:-1] + (gate.shape[-1],))
        up = up.reshape(shape[:-1] + (up.shape[-1],))
    return gate, up
