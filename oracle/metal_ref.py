"""Oracle (test infrastructure): ctypes access to oracle/_ref/libmetalref.so.

That library is the reference's own Metal kernel bodies compiled as C++ (see
metal_shim.cpp).  Each wrapper builds the int32 ``meta`` array the way the
reference's Python wrapper does (file:line in each docstring) and runs one
"thread" per grid position on the CPU.  Inputs and outputs are numpy arrays.
"""
from __future__ import annotations

import ctypes
import math
from pathlib import Path

import numpy as np

_LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libmetalref.so"
_lib = None


def available() -> bool:
    return _LIB_PATH.exists()


def _get():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(_LIB_PATH))
    return _lib


def _call(fn, *arrays_then_grid):
    """Calls ``fn`` with the data pointers of the arrays; the arrays stay referenced by this frame
    for the duration of the call (a bare pointer does not keep its array alive)."""
    *arrays, grid = arrays_then_grid
    for a in arrays:
        assert isinstance(a, np.ndarray) and a.flags["C_CONTIGUOUS"]
    fn(*[ctypes.c_void_p(a.ctypes.data) for a in arrays], ctypes.c_longlong(int(grid)))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(*vals):
    return np.asarray(vals, dtype=np.int32)


def _zeros_or_dummy(zeros, like):
    if zeros is None:
        return np.zeros_like(_f32(like)), 0
    return _f32(zeros), 1


def dequant(bits, codes, scales, zeros, group_size):
    """meta as in ops/quant_ops.py:246 (q4) / :309 (q8); fp16 output."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    M = codes.shape[0]
    K = codes.shape[1] * 2 if bits == 4 else codes.shape[1]
    z, has_zero = _zeros_or_dummy(zeros, scales)
    out = np.empty((M, K), dtype=np.float16)
    if bits == 4:
        meta = _i32(M, codes.shape[1], K, group_size, has_zero)
        _call(_get().ref_dequant_q4_f16, codes, _f32(scales), z, meta, out, M * K)
    else:
        meta = _i32(M, K, group_size, has_zero)
        _call(_get().ref_dequant_q8_f16, codes, _f32(scales), z, meta, out, M * K)
    return out


def matvec(bits, x, codes, scales, zeros, group_size):
    """Serial one-thread-per-output kernel; meta as in ops/quant_ops.py:564 (q4) / :624 (q8)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    B, K = x.shape
    N = codes.shape[0]
    z, has_zero = _zeros_or_dummy(zeros, scales)
    y = np.empty((B, N), dtype=np.float16)
    if bits == 4:
        meta = _i32(B, K, N, codes.shape[1], group_size, has_zero)
        _call(_get().ref_q4_matvec_f16, x, codes, _f32(scales), z, meta, y, B * N)
    else:
        meta = _i32(B, K, N, group_size, has_zero)
        _call(_get().ref_q8_matvec_f16, x, codes, _f32(scales), z, meta, y, B * N)
    return y


def paged_attention(bits, q, k_codes, v_codes, k_scales, v_scales, block_table, lengths, page_shape,
                    group_size, scale):
    """meta as in ops/paged_quantized_kv_ops.py:563-566 (q8) / :605-608 (q4); grid B*Hq."""
    q = np.ascontiguousarray(q, dtype=np.float16)
    B, _, Hq, D = q.shape
    num_pages, P, Hkv, _ = page_shape
    max_blocks = block_table.shape[1]
    groups = (D + group_size - 1) // group_size
    out = np.zeros_like(q)
    bt = np.ascontiguousarray(block_table, dtype=np.int32)
    ln = np.ascontiguousarray(lengths, dtype=np.int32)
    sc = np.asarray([scale], dtype=np.float32)
    args = [q, np.ascontiguousarray(k_codes, dtype=np.uint8), np.ascontiguousarray(v_codes, dtype=np.uint8),
            _f32(k_scales), _f32(v_scales), bt, ln]
    if bits == 4:
        meta = _i32(B, num_pages, P, max_blocks, Hq, Hkv, D, (D + 1) // 2, group_size, groups)
        _call(_get().ref_q4_paged_attn_f16, *args, meta, sc, out, B * Hq)
    else:
        meta = _i32(B, num_pages, P, max_blocks, Hq, Hkv, D, group_size, groups)
        _call(_get().ref_q8_paged_attn_f16, *args, meta, sc, out, B * Hq)
    return out


def contiguous_attention(bits, q, k_codes, v_codes, k_scales, v_scales, lengths, cache_shape, group_size, scale):
    """meta as in ops/quantized_kv_cache_ops.py:444-447 (q8) / :480-483 (q4); grid B*Hq."""
    q = np.ascontiguousarray(q, dtype=np.float16)
    B, _, Hq, D = q.shape
    _, max_s, Hkv, _ = cache_shape
    groups = (D + group_size - 1) // group_size
    out = np.zeros_like(q)
    ln = np.ascontiguousarray(lengths, dtype=np.int32)
    sc = np.asarray([scale], dtype=np.float32)
    args = [q, np.ascontiguousarray(k_codes, dtype=np.uint8), np.ascontiguousarray(v_codes, dtype=np.uint8),
            _f32(k_scales), _f32(v_scales), ln]
    if bits == 4:
        meta = _i32(B, max_s, Hq, Hkv, D, (D + 1) // 2, group_size, groups)
        _call(_get().ref_q4_attn_f16, *args, meta, sc, out, B * Hq)
    else:
        meta = _i32(B, max_s, Hq, Hkv, D, group_size, groups)
        _call(_get().ref_q8_attn_f16, *args, meta, sc, out, B * Hq)
    return out


def fused_swiglu(gate, up):
    """meta as in ops/activation_ops.py:144."""
    gate = np.ascontiguousarray(gate, dtype=np.float16)
    up = np.ascontiguousarray(up, dtype=np.float16)
    rows, dim = gate.shape
    out = np.empty_like(gate)
    _call(_get().ref_fused_swiglu_f16, gate, up, _i32(rows, dim), out, rows * dim)
    return out


def block_table_lookup(block_table, positions, page_size):
    """meta as in ops/paged_kv_ops.py:171."""
    bt = np.ascontiguousarray(block_table, dtype=np.int32)
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    B, max_blocks = bt.shape
    page_ids = np.empty((B,), dtype=np.int32)
    offsets = np.empty((B,), dtype=np.int32)
    _call(_get().ref_block_table_lookup, bt, pos, _i32(B, max_blocks, page_size), page_ids, offsets, B)
    return page_ids, offsets
