"""q4/q8 group-wise pack / dequant / matvec, CUDA backend.

Mirrors the public functions of the reference's ops/quant_ops.py (names, argument order,
defaults, validation order and error text).  Backend strings: ``"cuda"`` is the canonical name;
``"auto"`` and the reference's Metal names (``metal``, ``metal_parallel``, ``metal_tiled``) all
select the same CUDA kernels.  ``"reference"`` and the ``MLX_METAL_CI_SAFE_MODE=1`` switch ask
for the pure-MLX path, which this library does not contain: they raise
``ReferenceBackendUnavailable``.

Layout: q4 codes two per byte, low nibble = even k, ``[N, ceil(K/2)]`` uint8; q8 ``[N, K]``
uint8; ``scales`` / ``zeros`` ``[N, ceil(K/group_size)]``; dequantisation ``(q - zero) * scale``
or ``q * scale`` when ``zeros`` is None (ops/quant_ops.py:205-212).
"""
from __future__ import annotations

import math
import os

import torch

from . import _cabi

_OUT_DTYPES = (torch.float16, torch.bfloat16)
_MATVEC_BACKENDS = ("metal", "metal_parallel", "metal_tiled", "cuda")
_MATVEC_ERR = "backend must be one of 'reference', 'metal', 'metal_parallel', 'metal_tiled', 'auto', 'cuda'"
_DEQUANT_ERR = "backend must be one of 'reference', 'metal', 'auto', 'cuda'"


def _normalize_out_dtype(out_dtype):
    if out_dtype is None:
        return torch.float16
    if out_dtype not in _OUT_DTYPES:
        raise TypeError(f"out_dtype must be float16 or bfloat16, got {out_dtype}")
    return out_dtype


def _validate_group_params(M, K, scales, zeros, group_size):
    if group_size <= 0:
        raise ValueError("group_size must be positive")
    groups = math.ceil(K / group_size)
    if tuple(scales.shape) != (M, groups):
        raise ValueError(f"scales must have shape {(M, groups)}, got {tuple(scales.shape)}")
    if zeros is not None and tuple(zeros.shape) != (M, groups):
        raise ValueError(f"zeros must have shape {(M, groups)}, got {tuple(zeros.shape)}")
    return groups


# ---------------------------------------------------------------------------------------------
# packing (offline helpers; plain tensor ops on whatever device the codes live on)
# ---------------------------------------------------------------------------------------------
def pack_q4(q_unpacked: torch.Tensor) -> torch.Tensor:
    if q_unpacked.ndim != 2:
        raise ValueError(f"q_unpacked must be 2-D [M,K], got {tuple(q_unpacked.shape)}")
    q_int = q_unpacked.to(torch.uint8)
    if q_int.shape[1] % 2 != 0:
        q_int = torch.nn.functional.pad(q_int, (0, 1))
    return (q_int[:, 0::2] + (q_int[:, 1::2] << 4)).to(torch.uint8).contiguous()


def unpack_q4_reference(packed: torch.Tensor, K: int | None = None) -> torch.Tensor:
    if packed.ndim != 2:
        raise ValueError(f"packed must be 2-D [M,K_packed], got {tuple(packed.shape)}")
    p = packed.to(torch.uint8)
    out = torch.stack([p & 0x0F, (p >> 4) & 0x0F], dim=-1).reshape(p.shape[0], p.shape[1] * 2)
    if K is not None:
        out = out[:, :K]
    return out.to(torch.uint8)


# ---------------------------------------------------------------------------------------------
# dequant
# ---------------------------------------------------------------------------------------------
def dequant_codes(bits, codes, scales, zeros, M, K, group_size, out_dtype):
    """Launcher shared with the paged-KV module: codes [M, row_bytes] -> [M, K]."""
    _cabi.require_cuda(codes, scales, zeros)
    codes = _cabi.contiguous(codes.to(torch.uint8))
    scales, zeros = _cabi.scale_pair(scales, zeros)
    out = torch.empty((M, K), dtype=out_dtype, device=codes.device)
    _cabi.check(
        _cabi.load().b200q_dequant(bits, codes.data_ptr(), scales.data_ptr(), _cabi.ptr(zeros), out.data_ptr(), M, K,
                                   group_size, _cabi.dtype_code(scales.dtype), _cabi.dtype_code(out_dtype),
                                   _cabi.stream()),
        "b200q_dequant",
    )
    return out


def _dequant(bits, q, scales, zeros, group_size, out_dtype, backend, who):
    if q.ndim != 2:
        what = "packed must be 2-D [M,K_packed]" if bits == 4 else "q must be 2-D [M,K]"
        raise ValueError(f"{what}, got {tuple(q.shape)}")
    out_dtype = _normalize_out_dtype(out_dtype)
    M = q.shape[0]
    K = q.shape[1] * 2 if bits == 4 else q.shape[1]
    _validate_group_params(M, K, scales, zeros, group_size)
    name = backend.lower()
    if name == "auto":
        name = "cuda"
    if _cabi.safe_mode_enabled() or name == "reference":
        _cabi.reference_unavailable(who)
    if name not in ("metal", "cuda"):
        raise ValueError(_DEQUANT_ERR)
    return dequant_codes(bits, q, scales, zeros, M, K, group_size, out_dtype)


def reference_dequant_q4(packed, scales, zeros=None, *, group_size: int = 32, out_dtype=None):
    _cabi.reference_unavailable("reference_dequant_q4")


def reference_dequant_q8(q, scales, zeros=None, *, group_size: int = 32, out_dtype=None):
    _cabi.reference_unavailable("reference_dequant_q8")


def dequant_q4(packed, scales, zeros=None, *, group_size: int = 32, out_dtype=None, backend: str = "auto"):
    """Bit-exact ``cast((q - zero) * scale)`` (ops/quant_ops.py:215-253)."""
    return _dequant(4, packed, scales, zeros, group_size, out_dtype, backend, "dequant_q4")


def dequant_q8(q, scales, zeros=None, *, group_size: int = 32, out_dtype=None, backend: str = "auto"):
    """ops/quant_ops.py:279-316."""
    return _dequant(8, q, scales, zeros, group_size, out_dtype, backend, "dequant_q8")


def groupwise_dequant(q, scales, zeros=None, *, bits, group_size: int = 32, out_dtype=None, backend: str = "auto"):
    if bits == 4:
        return dequant_q4(q, scales, zeros, group_size=group_size, out_dtype=out_dtype, backend=backend)
    if bits == 8:
        return dequant_q8(q, scales, zeros, group_size=group_size, out_dtype=out_dtype, backend=backend)
    raise ValueError(f"bits must be 4 or 8, got {bits}")


# ---------------------------------------------------------------------------------------------
# matvec
# ---------------------------------------------------------------------------------------------
def _normalize_x_2d(x):
    if x.ndim == 2:
        return x, x.shape[0], x.shape[1]
    if x.ndim == 3 and x.shape[1] == 1:
        squeezed = x[:, 0, :]
        return squeezed, squeezed.shape[0], squeezed.shape[1]
    raise ValueError(f"x must have shape [B,K] or [B,1,K], got {tuple(x.shape)}")


def _validate_matvec_input_dtype(x2d):
    if x2d.dtype not in _OUT_DTYPES:
        raise TypeError(f"x dtype must be float16 or bfloat16, got {x2d.dtype}")


def _normalize_hidden_rows_input(x):
    if x.ndim == 2:
        return x, tuple(x.shape), x.shape[0], x.shape[1]
    if x.ndim == 3:
        rows = x.shape[0] * x.shape[1]
        return x.reshape(rows, x.shape[2]), tuple(x.shape), rows, x.shape[2]
    raise ValueError(f"x must have shape [rows,K] or [B,S,K], got {tuple(x.shape)}")


def _restore_hidden_rows_output(y2d, original_shape):
    if len(original_shape) == 2:
        return y2d
    return y2d.reshape(original_shape[:-1] + (y2d.shape[-1],))


def matvec_rows(bits, x2d, codes, scales, zeros, group_size, residual=None):
    """Launcher: x2d [B,K] -> [B,N]; with ``residual`` [B,N] returns cast(residual + cast(y))."""
    _cabi.require_cuda(x2d, codes, scales, zeros, residual)
    x2d = _cabi.contiguous(x2d)
    codes = _cabi.contiguous(codes.to(torch.uint8))
    scales, zeros = _cabi.scale_pair(scales, zeros)
    residual = None if residual is None else _cabi.contiguous(residual.to(x2d.dtype))
    B, K = x2d.shape
    N = codes.shape[0]
    y = torch.empty((B, N), dtype=x2d.dtype, device=x2d.device)
    _cabi.check(
        _cabi.load().b200q_qmatvec(bits, x2d.data_ptr(), codes.data_ptr(), scales.data_ptr(), _cabi.ptr(zeros),
                                   _cabi.ptr(residual), y.data_ptr(), B, N, K, group_size,
                                   _cabi.dtype_code(x2d.dtype), _cabi.dtype_code(scales.dtype), _cabi.stream()),
        "b200q_qmatvec",
    )
    return y


def _resolve_matvec_backend(backend: str, who: str) -> None:
    name = backend.lower()
    if name == "auto":
        # the reference picks metal or metal_tiled from MLX_METAL_USE_TILED_MATVEC; both are the CUDA kernel here
        name = "metal_tiled" if os.environ.get("MLX_METAL_USE_TILED_MATVEC", "0") == "1" else "metal"
    if name == "reference":
        _cabi.reference_unavailable(who)
    if _cabi.safe_mode_enabled():
        _cabi.reference_unavailable(who)
    if name not in _MATVEC_BACKENDS:
        raise ValueError(_MATVEC_ERR)


def reference_q4_matvec_decode(x, packed_w, scales, zeros=None, *, group_size: int = 32):
    _cabi.reference_unavailable("reference_q4_matvec_decode")


def reference_q8_matvec_decode(x, q_w, scales, zeros=None, *, group_size: int = 32):
    _cabi.reference_unavailable("reference_q8_matvec_decode")


def q4_matvec_decode(x, packed_w, scales, zeros=None, *, group_size: int = 32, backend: str = "auto"):
    """x [B,K] or [B,1,K] -> [B,N] in x.dtype (ops/quant_ops.py:529-571)."""
    x2d, B, K = _normalize_x_2d(x)
    _validate_matvec_input_dtype(x2d)
    if packed_w.ndim != 2:
        raise ValueError(f"packed_w must be 2-D [N,K_packed], got {tuple(packed_w.shape)}")
    N, K_packed = packed_w.shape
    if K_packed * 2 != K:
        raise ValueError(f"packed_w implies K={K_packed * 2}, but x has K={K}")
    _validate_group_params(N, K, scales, zeros, group_size)
    _resolve_matvec_backend(backend, "q4_matvec_decode")
    return matvec_rows(4, x2d, packed_w, scales, zeros, group_size)


def q8_matvec_decode(x, q_w, scales, zeros=None, *, group_size: int = 32, backend: str = "auto"):
    """ops/quant_ops.py:591-631."""
    x2d, B, K = _normalize_x_2d(x)
    _validate_matvec_input_dtype(x2d)
    if q_w.ndim != 2 or q_w.shape[1] != K:
        raise ValueError(f"q_w must have shape [N,{K}], got {tuple(q_w.shape)}")
    N = q_w.shape[0]
    _validate_group_params(N, K, scales, zeros, group_size)
    _resolve_matvec_backend(backend, "q8_matvec_decode")
    return matvec_rows(8, x2d, q_w, scales, zeros, group_size)


# ---------------------------------------------------------------------------------------------
# gate / up in one launch
# ---------------------------------------------------------------------------------------------
def _validate_gate_up_shapes(x2d, gate_w, up_w, gate_scales, up_scales, gate_zeros, up_zeros, *, bits, group_size):
    _validate_matvec_input_dtype(x2d)
    if bits not in (4, 8):
        raise ValueError(f"bits must be 4 or 8, got {bits}")
    rows, k_dim = x2d.shape
    if gate_w.ndim != 2 or up_w.ndim != 2:
        raise ValueError(f"gate_w and up_w must be 2-D, got {tuple(gate_w.shape)}, {tuple(up_w.shape)}")
    if gate_w.shape != up_w.shape:
        raise ValueError(f"gate_w and up_w must have identical shapes, got {tuple(gate_w.shape)}, {tuple(up_w.shape)}")
    out_dim = gate_w.shape[0]
    if bits == 4:
        expected_cols = math.ceil(k_dim / 2)
        if gate_w.shape[1] != expected_cols:
            raise ValueError(f"q4 gate/up weights must have shape [{out_dim},{expected_cols}], got {tuple(gate_w.shape)}")
    elif gate_w.shape[1] != k_dim:
        raise ValueError(f"q8 gate/up weights must have shape [{out_dim},{k_dim}], got {tuple(gate_w.shape)}")
    groups = _validate_group_params(out_dim, k_dim, gate_scales, gate_zeros, group_size)
    up_groups = _validate_group_params(out_dim, k_dim, up_scales, up_zeros, group_size)
    if groups != up_groups:
        raise ValueError(f"gate and up scale group counts must match, got {groups} and {up_groups}")
    return rows, k_dim, out_dim


def gate_up_rows(bits, x2d, gate_w, up_w, gate_scales, up_scales, gate_zeros, up_zeros, group_size, *,
                 want_gate_up=True, want_act=False, residual_in=None, norm_weight=None, eps=1e-5, want_z=False,
                 want_normed=False):
    """Launcher of the fused gate/up (+ optional RMSNorm prologue, + SwiGLU) kernel on rows [R,K].
    Returns a dict with the requested tensors among gate, up, act, z, normed."""
    _cabi.require_cuda(x2d, gate_w, up_w, gate_scales, up_scales, gate_zeros, up_zeros, residual_in, norm_weight)
    x2d = _cabi.contiguous(x2d)
    gate_w = _cabi.contiguous(gate_w.to(torch.uint8))
    up_w = _cabi.contiguous(up_w.to(torch.uint8))
    # one scale dtype for the launch
    all_sz = [t for t in (gate_scales, up_scales, gate_zeros, up_zeros) if t is not None]
    dt = all_sz[0].dtype
    if dt not in (torch.float16, torch.bfloat16, torch.float32) or any(t.dtype != dt for t in all_sz):
        dt = torch.float32
    conv = lambda t: None if t is None else _cabi.contiguous(t.to(dt))
    gate_scales, up_scales, gate_zeros, up_zeros = conv(gate_scales), conv(up_scales), conv(gate_zeros), conv(up_zeros)
    if (gate_zeros is None) != (up_zeros is None):
        # the kernel takes the zero-point term per matrix; a missing one is simply absent
        pass
    R, K = x2d.shape
    N = gate_w.shape[0]
    dev, adt = x2d.device, x2d.dtype
    new = lambda *shape: torch.empty(shape, dtype=adt, device=dev)
    out = {}
    if want_gate_up:
        out["gate"], out["up"] = new(R, N), new(R, N)
    if want_act:
        out["act"] = new(R, N)
    if norm_weight is not None:
        norm_weight = _cabi.contiguous(norm_weight)
        residual_in = None if residual_in is None else _cabi.contiguous(residual_in.to(adt))
        if want_z:
            out["z"] = new(R, K)
        # the generic (odd-shape) route needs the normalised rows as a buffer, so always provide it
        out["normed"] = new(R, K)
    _cabi.check(
        _cabi.load().b200q_gate_up_swiglu(
            bits, x2d.data_ptr(), gate_w.data_ptr(), up_w.data_ptr(), gate_scales.data_ptr(), up_scales.data_ptr(),
            _cabi.ptr(gate_zeros), _cabi.ptr(up_zeros), _cabi.ptr(out.get("gate")), _cabi.ptr(out.get("up")),
            _cabi.ptr(out.get("act")), _cabi.ptr(residual_in), _cabi.ptr(norm_weight),
            _cabi.dtype_code(norm_weight.dtype) if norm_weight is not None else _cabi.F16, float(eps),
            _cabi.ptr(out.get("z")), _cabi.ptr(out.get("normed")), R, N, K, group_size, _cabi.dtype_code(adt),
            _cabi.dtype_code(dt), _cabi.stream()),
        "b200q_gate_up_swiglu",
    )
    if not want_normed:
        out.pop("normed", None)
    return out


def _gate_up_matvec_tiled(bits, x, gate_w, up_w, gate_scales, up_scales, gate_zeros, up_zeros, group_size):
    x2d, original_shape, rows, k_dim = _normalize_hidden_rows_input(x)
    _validate_gate_up_shapes(x2d, gate_w, up_w, gate_scales, up_scales, gate_zeros, up_zeros, bits=bits,
                             group_size=group_size)
    res = gate_up_rows(bits, x2d, gate_w, up_w, gate_scales, up_scales, gate_zeros, up_zeros, group_size)
    return (_restore_hidden_rows_output(res["gate"], original_shape),
            _restore_hidden_rows_output(res["up"], original_shape))


def q4_gate_up_matvec_tiled(x, gate_packed, up_packed, gate_scales, up_scales, gate_zeros=None, up_zeros=None, *,
                            group_size: int = 32):
    """(gate, up) projections of the same rows in one launch (ops/quant_ops.py:634-685)."""
    return _gate_up_matvec_tiled(4, x, gate_packed, up_packed, gate_scales, up_scales, gate_zeros, up_zeros, group_size)


def q8_gate_up_matvec_tiled(x, gate_q, up_q, gate_scales, up_scales, gate_zeros=None, up_zeros=None, *,
                            group_size: int = 32):
    """ops/quant_ops.py:688-738."""
    return _gate_up_matvec_tiled(8, x, gate_q, up_q, gate_scales, up_scales, gate_zeros, up_zeros, group_size)
