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


# ---------------------------------------------------------------------------------------------
# bodies pinned since the threadgroup emulator exists (metal_shim.cpp, second half)
# ---------------------------------------------------------------------------------------------
def _call_tg(fn, *arrays_then_groups_threads):
    *arrays, groups, threads = arrays_then_groups_threads
    for a in arrays:
        assert isinstance(a, np.ndarray) and a.flags["C_CONTIGUOUS"]
    fn(*[ctypes.c_void_p(a.ctypes.data) for a in arrays], ctypes.c_longlong(int(groups)), ctypes.c_longlong(int(threads)))


def residual_add(x, residual):
    """kernels/residual_add.metal; meta as in ops/fused_ops.py:168-180 (total element count)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    r = np.ascontiguousarray(residual, dtype=np.float16)
    y = np.empty_like(x)
    _call(_get().ref_residual_add_f16, x, r, _i32(x.size), y, x.size)
    return y


def swiglu(gate, up):
    """kernels/swiglu.metal; gate/up [B,S,D], meta = (B, S, D) as in ops/activation_ops.py:112-123."""
    gate = np.ascontiguousarray(gate, dtype=np.float16)
    up = np.ascontiguousarray(up, dtype=np.float16)
    B, S, D = gate.shape
    out = np.empty_like(gate)
    _call(_get().ref_swiglu_f16, gate, up, _i32(B, S, D), out, gate.size)
    return out


def rms_norm(x, weight, eps, threads=256):
    """kernels/rms_norm.metal: one threadgroup of 256 threads per row, meta = (B, S, D) (ops/norm_ops.py:12,76-85)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    w = np.ascontiguousarray(weight, dtype=np.float16)
    B, S, D = x.shape
    y = np.empty_like(x)
    _call_tg(_get().ref_rms_norm_f16, x, w, _i32(B, S, D), np.asarray([eps], dtype=np.float32), y, B * S, threads)
    return y


def rmsnorm_residual(x, residual, weight, eps, threads=256):
    """kernels/rmsnorm_residual.metal: (y, z), meta = (rows, D), 256 threads per row (ops/fused_ops.py:16,228-240)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    r = np.ascontiguousarray(residual, dtype=np.float16)
    w = np.ascontiguousarray(weight, dtype=np.float16)
    D = x.shape[-1]
    rows = x.size // D
    y, z = np.empty_like(x), np.empty_like(x)
    _call_tg(_get().ref_rmsnorm_residual_f16, x, r, w, _i32(rows, D), np.asarray([eps], dtype=np.float32), y, z, rows,
             threads)
    return y, z


def matvec_parallel(bits, x, codes, scales, zeros, group_size, threads=128):
    """kernels/q{4,8}_matvec_decode_parallel.metal: one threadgroup of 128 threads per output
    (ops/quant_ops.py:24, meta as built for the ``metal_parallel`` backend)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    B, K = x.shape
    N = codes.shape[0]
    groups = (K + group_size - 1) // group_size
    z, has_zero = _zeros_or_dummy(zeros, scales)
    y = np.empty((B, N), dtype=np.float16)
    if bits == 4:
        meta = _i32(B, N, K, codes.shape[1], group_size, groups, has_zero)
        _call_tg(_get().ref_q4_matvec_parallel_f16, x, codes, _f32(scales), z, meta, y, B * N, threads)
    else:
        meta = _i32(B, N, K, group_size, groups, has_zero)
        _call_tg(_get().ref_q8_matvec_parallel_f16, x, codes, _f32(scales), z, meta, y, B * N, threads)
    return y


def matvec_tiled(bits, x, codes, scales, zeros, group_size, n_tile=4, threads=128):
    """kernels/q{4,8}_matvec_decode_tiled.metal: four outputs per threadgroup of 128 threads
    (ops/quant_ops.py:25-26, 457-480)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    B, K = x.shape
    N = codes.shape[0]
    groups = (K + group_size - 1) // group_size
    tiles = B * ((N + n_tile - 1) // n_tile)
    z, has_zero = _zeros_or_dummy(zeros, scales)
    y = np.empty((B, N), dtype=np.float16)
    if bits == 4:
        meta = _i32(B, N, K, codes.shape[1], group_size, groups, has_zero, n_tile)
        _call_tg(_get().ref_q4_matvec_tiled_f16, x, codes, _f32(scales), z, meta, y, tiles, threads)
    else:
        meta = _i32(B, N, K, group_size, groups, has_zero, n_tile)
        _call_tg(_get().ref_q8_matvec_tiled_f16, x, codes, _f32(scales), z, meta, y, tiles, threads)
    return y


def gate_up_tiled(bits, x, gate_codes, up_codes, gate_scales, up_scales, gate_zeros, up_zeros, group_size, n_tile=4,
                  threads=128):
    """kernels/q{4,8}_gate_up_matvec_tiled.metal: (gate, up) rows (ops/quant_ops.py:634-738)."""
    x = np.ascontiguousarray(x, dtype=np.float16)
    gc = np.ascontiguousarray(gate_codes, dtype=np.uint8)
    uc = np.ascontiguousarray(up_codes, dtype=np.uint8)
    rows, K = x.shape
    N = gc.shape[0]
    groups = (K + group_size - 1) // group_size
    tiles = rows * ((N + n_tile - 1) // n_tile)
    gz, has_gz = _zeros_or_dummy(gate_zeros, gate_scales)
    uz, has_uz = _zeros_or_dummy(up_zeros, up_scales)
    gate = np.empty((rows, N), dtype=np.float16)
    up = np.empty((rows, N), dtype=np.float16)
    if bits == 4:
        meta = _i32(rows, K, N, gc.shape[1], group_size, groups, has_gz, has_uz, n_tile)
        fn = _get().ref_q4_gate_up_tiled_f16
    else:
        meta = _i32(rows, K, N, group_size, groups, has_gz, has_uz, n_tile)
        fn = _get().ref_q8_gate_up_tiled_f16
    _call_tg(fn, x, gc, uc, _f32(gate_scales), _f32(up_scales), gz, uz, meta, gate, up, tiles, threads)
    return gate, up
