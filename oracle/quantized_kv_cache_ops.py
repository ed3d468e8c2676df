"""Oracle (test infrastructure): contiguous q4/q8 KV cache and its GQA decode attention.

Vectorised restatement of ops/quantized_kv_cache_ops.py.  The reference loops in Python over
every (batch, head, token, group); the arithmetic per group is the same symmetric scale-only rule
as the paged cache and is reproduced here on whole tensors.  Layout: codes
``[B, MAX_S, Hkv, D]`` (q8) or ``[.., ceil(D/2)]`` (q4, low nibble = even d), scales
``[B, MAX_S, Hkv, ceil(D/group_size)]`` fp16.  Only the shipped package's tests import this.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch

from .paged_kv_ops import normalize_positions, validate_gqa_heads
from .paged_quantized_kv_ops import _quantize_groups_symmetric
from .quant_ops import pack_q4, unpack_q4_reference


@dataclass
class OracleQuantizedKV:
    """Field-for-field twin of QuantizedKVCache (ops/quantized_kv_cache_ops.py:69-81)."""
    k_q: Any
    v_q: Any
    k_scales: Any
    v_scales: Any
    k_zeros: Any | None = None
    v_zeros: Any | None = None
    bits: int = 8
    group_size: int = 32
    original_shape: tuple[int, ...] | None = None
    layout: str = "contiguous"
    metadata: dict[str, Any] = field(default_factory=dict)


def quantize_kv_cache(K_cache, V_cache, *, bits=8, group_size=32, lengths=None):
    """ops/quantized_kv_cache_ops.py:173-277: tokens below ``lengths[b]`` are quantised group by
    group; everything at or past the length keeps code 0 and scale 0."""
    if bits not in (4, 8):
        raise ValueError(f"bits must be 4 or 8, got {bits}")
    if K_cache.shape != V_cache.shape:
        raise ValueError(f"K_cache and V_cache must match, got {tuple(K_cache.shape)} != {tuple(V_cache.shape)}")
    if K_cache.ndim != 4:
        raise ValueError(f"K_cache must be 4-D [B,MAX_S,Hkv,D], got {tuple(K_cache.shape)}")
    B, MAX_S, Hkv, D = K_cache.shape
    if lengths is not None:
        lengths_arr = normalize_positions(lengths, B, MAX_S + 1).to(torch.int64)
    else:
        lengths_arr = torch.full((B,), MAX_S, dtype=torch.int64)
    valid = (torch.arange(MAX_S).reshape(1, MAX_S) < lengths_arr.reshape(B, 1)).reshape(B, MAX_S, 1, 1)
    limit, offset = (127, 128) if bits == 8 else (7, 8)
    out = {}
    for name, cache in (("k", K_cache), ("v", V_cache)):
        codes, scales = _quantize_groups_symmetric(cache.to(torch.float32), group_size, limit, offset)
        codes = torch.where(valid, codes, torch.zeros_like(codes))
        scales = torch.where(valid, scales, torch.zeros_like(scales))
        if bits == 4:
            codes = pack_q4(codes.reshape(-1, D)).reshape(B, MAX_S, Hkv, (D + 1) // 2)
        out[name] = (codes.contiguous(), scales.contiguous())
    return OracleQuantizedKV(k_q=out["k"][0], v_q=out["v"][0], k_scales=out["k"][1], v_scales=out["v"][1],
                             bits=bits, group_size=group_size, original_shape=tuple(K_cache.shape))


def _cache_dims(cache):
    """ops/quantized_kv_cache_ops.py:282-283, 358-365: the original shape, else read off the codes."""
    if cache.original_shape is not None:
        return tuple(cache.original_shape)
    B, MAX_S, Hkv, last = cache.k_q.shape
    return B, MAX_S, Hkv, (last if cache.bits == 8 else last * 2)


def _dequant(codes_q, scales, bits, group_size, shape):
    """_dequant_group_symmetric_8/_4 + cast (ops/quantized_kv_cache_ops.py:141-170, 289-311):
    (code - 128|8) * |scale| in fp32, then fp16."""
    B, MAX_S, Hkv, D = shape
    if bits == 4:
        codes = unpack_q4_reference(codes_q.reshape(-1, codes_q.shape[-1]), K=D).reshape(B, MAX_S, Hkv, D)
        signed = codes.to(torch.float32) - 8.0
    else:
        signed = codes_q.to(torch.float32) - 128.0
    scale_expanded = scales.to(torch.float32).repeat_interleave(group_size, dim=-1)[..., :D]
    return (signed * scale_expanded.abs()).to(torch.float16)


def dequantize_kv_cache(cache):
    """ops/quantized_kv_cache_ops.py:280-313."""
    shape = _cache_dims(cache)
    return (_dequant(cache.k_q, cache.k_scales, cache.bits, cache.group_size, shape),
            _dequant(cache.v_q, cache.v_scales, cache.bits, cache.group_size, shape))


def reference_quantized_kv_gqa_decode_attention(q, cache, lengths=None, *, scale=None, window=None):
    """ops/quantized_kv_cache_ops.py:348-406: K and V dequantised and rounded to fp16, scores in
    fp32, positions at or past the length get -1e9 before the softmax over all MAX_S positions,
    result cast to q.dtype.  (With one valid token or more the masked terms are exactly 0 in fp32,
    so this is the softmax over the valid tokens; a length of 0 averages all MAX_S positions.)

    ``window=(sink, recent)`` keeps only the first ``sink`` and the last ``recent`` valid positions: the decode
    row of the sliding_window(_sink) masks that reference_quantized_kv_sparse_gqa_decode_attention applies
    (ops/quantized_kv_cache_ops.py:544-583); ``None`` means dense."""
    if q.ndim != 4:
        raise ValueError(f"q must be 4-D [B,1,Hq,D], got {tuple(q.shape)}")
    if q.shape[1] != 1:
        raise ValueError(f"q must have shape [B,1,Hq,D], got {tuple(q.shape)}")
    B, _, Hq, D = q.shape
    cache_B, MAX_S, Hkv, D_cache = _cache_dims(cache)
    if B != cache_B:
        raise ValueError(f"batch mismatch: q batch={B}, cache batch={cache_B}")
    if D != D_cache:
        raise ValueError(f"head_dim mismatch: q D={D}, cache D={D_cache}")
    validate_gqa_heads(Hq, Hkv)
    lengths_arr = normalize_positions(lengths if lengths is not None else MAX_S, B, MAX_S + 1).to(torch.int64)
    lengths_arr = torch.clamp(lengths_arr, max=MAX_S)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    K_deq, V_deq = dequantize_kv_cache(cache)
    Kf, Vf, qf = K_deq.to(torch.float32), V_deq.to(torch.float32), q.to(torch.float32)
    group = Hq // Hkv
    qg = qf[:, 0].reshape(B, Hkv, group, D)
    scores = torch.einsum("bhgd,bshd->bhgs", qg, Kf) * float(scale)
    valid = (torch.arange(MAX_S).reshape(1, 1, 1, MAX_S) < lengths_arr.reshape(B, 1, 1, 1))
    if window is not None:
        sink, recent = window
        pos = torch.arange(MAX_S).reshape(1, 1, 1, MAX_S)
        valid = valid & ((pos < sink) | (pos >= (lengths_arr - recent).reshape(B, 1, 1, 1)))
    scores = torch.where(valid, scores, torch.full_like(scores, -1.0e9))
    probs = torch.softmax(scores, dim=-1)
    out = torch.einsum("bhgs,bshd->bhgd", probs, Vf).reshape(B, 1, Hq, D)
    return out.to(q.dtype)
