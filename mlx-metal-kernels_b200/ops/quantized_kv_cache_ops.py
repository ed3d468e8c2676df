"""Contiguous quantized KV cache (q8 / q4, symmetric, fp16 scales) and its GQA decode attention.

Mirrors ops/quantized_kv_cache_ops.py of the reference: the config and cache dataclasses, cache
quantise / dequantise, the error report and the decode-attention entry point.
Layouts: codes ``[B, MAX_S, Hkv, D]`` (q8) or ``[.., ceil(D/2)]`` (q4, low nibble = even d), scales
``[B, MAX_S, Hkv, ceil(D/group_size)]`` fp16.

A contiguous cache is a paged cache whose block table is the identity, so the attention runs on the
paged split-KV kernels without copying anything: with MAX_S a multiple of 16 the buffers are viewed
as ``B * MAX_S / 16`` pages of 16 tokens; otherwise every sequence is one page of MAX_S tokens (the
general kernel).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch

from . import _cabi
from .gqa_ops import validate_gqa_heads
from .paged_kv_ops import normalize_positions
from .paged_quantized_kv_ops import PagedQuantizedKVCache, _quantize_groups, paged_attention_launch
from .quant_ops import dequant_codes
from .sparse_attention_ops import SparseAttentionPattern, decode_block_mask, decode_window

_MAX_HEAD_DIM = 128
_FAST_PAGE = 16


def _dtype_itemsize(dtype: Any) -> int:
    return torch.empty((), dtype=dtype).element_size()


@dataclass
class QuantizedKVCacheConfig:
    bits: int = 8
    group_size: int = 32
    symmetric: bool = True
    with_zeros: bool = False
    scale_dtype: str = "float16"
    layout: str = "contiguous"

    def validate(self) -> "QuantizedKVCacheConfig":
        if self.bits not in (4, 8):
            raise ValueError(f"bits must be 4 or 8, got {self.bits}")
        if self.group_size <= 0:
            raise ValueError(f"group_size must be > 0, got {self.group_size}")
        if not self.symmetric:
            raise NotImplementedError("asymmetric quantization is not implemented yet")
        if self.with_zeros:
            raise NotImplementedError("zero-point quantization is not implemented yet")
        if self.layout != "contiguous":
            raise NotImplementedError(f"layout={self.layout!r} is not implemented yet; use 'contiguous'")
        return self


@dataclass
class QuantizedKVCache:
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

    def shapes(self) -> dict[str, tuple[int, ...] | None]:
        return {
            "k_q": tuple(self.k_q.shape),
            "v_q": tuple(self.v_q.shape),
            "k_scales": tuple(self.k_scales.shape),
            "v_scales": tuple(self.v_scales.shape),
            "original": None if self.original_shape is None else tuple(self.original_shape),
        }

    def validate(self) -> "QuantizedKVCache":
        if self.bits not in (4, 8):
            raise ValueError(f"bits must be 4 or 8, got {self.bits}")
        if self.k_q.shape != self.v_q.shape:
            raise ValueError(f"k_q and v_q shapes must match, got {tuple(self.k_q.shape)} != {tuple(self.v_q.shape)}")
        if self.k_scales.shape != self.v_scales.shape:
            raise ValueError(f"k_scales and v_scales shapes must match, got {tuple(self.k_scales.shape)} != {tuple(self.v_scales.shape)}")
        if self.layout != "contiguous":
            raise NotImplementedError(f"layout={self.layout!r} is not supported")
        if self.original_shape is not None and len(self.original_shape) != 4:
            raise ValueError(f"original_shape must be 4-D [B,MAX_S,Hkv,D], got {self.original_shape}")
        return self

    def memory_bytes(self) -> int:
        total = 0
        for arr in (self.k_q, self.v_q, self.k_scales, self.v_scales, self.k_zeros, self.v_zeros):
            if arr is not None:
                total += arr.numel() * _dtype_itemsize(arr.dtype)
        return total

    def compression_ratio(self, fp_bytes_per_value: int = 2) -> float | None:
        if self.original_shape is None:
            return None
        B, MAX_S, Hkv, D = self.original_shape
        fp_bytes = 2 * B * MAX_S * Hkv * D * fp_bytes_per_value
        q_bytes = self.memory_bytes()
        return None if q_bytes == 0 else fp_bytes / q_bytes


def _cache_dims(qkv_cache: QuantizedKVCache) -> tuple[int, int, int, int]:
    if qkv_cache.original_shape is not None:
        B, MAX_S, Hkv, D = qkv_cache.original_shape
        return int(B), int(MAX_S), int(Hkv), int(D)
    B, MAX_S, Hkv, last = qkv_cache.k_q.shape
    return B, MAX_S, Hkv, (last if qkv_cache.bits == 8 else last * 2)


# ---------------------------------------------------------------------------------------------
# quantise / dequantise
# ---------------------------------------------------------------------------------------------
def quantize_kv_cache(K_cache, V_cache, config: QuantizedKVCacheConfig, *, lengths=None) -> QuantizedKVCache:
    """fp16/bf16 caches [B,MAX_S,Hkv,D] -> quantized cache (ops/quantized_kv_cache_ops.py:173-277).
    Tokens at or past ``lengths[b]`` keep code 0 and scale 0, as in the reference.  The group
    quantisation runs in the CUDA kernel behind b200q_quantize_kv; the length mask is a tensor op."""
    config = config.validate()
    if K_cache.shape != V_cache.shape:
        raise ValueError(f"K_cache and V_cache must match, got {tuple(K_cache.shape)} != {tuple(V_cache.shape)}")
    if K_cache.ndim != 4:
        raise ValueError(f"K_cache must be 4-D [B,MAX_S,Hkv,D], got {tuple(K_cache.shape)}")
    B, MAX_S, Hkv, D = K_cache.shape
    valid = None
    if lengths is not None:
        lengths_arr = normalize_positions(lengths, B, MAX_S + 1, device=K_cache.device)
        valid = (torch.arange(MAX_S, device=K_cache.device).reshape(1, MAX_S) < lengths_arr.reshape(B, 1))
        valid = valid.reshape(B, MAX_S, 1, 1)
    out = []
    for cache in (K_cache, V_cache):
        codes, scales = _quantize_groups(cache, config.bits, config.group_size)
        if valid is not None:
            codes = torch.where(valid, codes, torch.zeros_like(codes))
            scales = torch.where(valid, scales, torch.zeros_like(scales))
        out.append((codes.contiguous(), scales.contiguous()))      # q4 codes come packed from the kernel
    return QuantizedKVCache(k_q=out[0][0], v_q=out[1][0], k_scales=out[0][1], v_scales=out[1][1],
                            bits=config.bits, group_size=config.group_size, original_shape=tuple(K_cache.shape),
                            layout=config.layout)


def dequantize_kv_cache(qkv_cache: QuantizedKVCache):
    """(K, V) fp16 [B,MAX_S,Hkv,D] = cast((code - 128|8) * |scale|)
    (ops/quantized_kv_cache_ops.py:280-313), through the bit-exact dequant kernel."""
    qkv_cache = qkv_cache.validate()
    B, MAX_S, Hkv, D = _cache_dims(qkv_cache)
    rows = B * MAX_S * Hkv
    groups = (D + qkv_cache.group_size - 1) // qkv_cache.group_size
    offset = 128.0 if qkv_cache.bits == 8 else 8.0
    outs = []
    for codes, scales in ((qkv_cache.k_q, qkv_cache.k_scales), (qkv_cache.v_q, qkv_cache.v_scales)):
        s = scales.reshape(rows, groups).abs()
        z = torch.full_like(s, offset)
        out = dequant_codes(qkv_cache.bits, codes.reshape(rows, codes.shape[-1]), s, z, rows, D,
                            qkv_cache.group_size, torch.float16)
        outs.append(out.reshape(B, MAX_S, Hkv, D))
    return outs[0], outs[1]


def quantized_kv_error(K_cache, V_cache, qkv_cache: QuantizedKVCache) -> dict[str, float]:
    """Error report of a quantised cache against its source (ops/quantized_kv_cache_ops.py:316-340)."""
    K_deq, V_deq = dequantize_kv_cache(qkv_cache)
    k_diff = K_cache.to(torch.float32) - K_deq.to(torch.float32)
    v_diff = V_cache.to(torch.float32) - V_deq.to(torch.float32)
    cr = qkv_cache.compression_ratio(fp_bytes_per_value=2)
    return {
        "k_max_abs_error": float(k_diff.abs().max()),
        "k_mean_abs_error": float(k_diff.abs().mean()),
        "k_rmse": float(k_diff.pow(2).mean().sqrt()),
        "v_max_abs_error": float(v_diff.abs().max()),
        "v_mean_abs_error": float(v_diff.abs().mean()),
        "v_rmse": float(v_diff.pow(2).mean().sqrt()),
        "compression_ratio": float(cr) if cr is not None else 0.0,
    }


# ---------------------------------------------------------------------------------------------
# decode attention
# ---------------------------------------------------------------------------------------------
def _validate_quantized_decode_inputs(q, qkv_cache: QuantizedKVCache, lengths):
    if q.ndim != 4:
        raise ValueError(f"q must be 4-D [B,1,Hq,D], got {tuple(q.shape)}")
    if q.shape[1] != 1:
        raise ValueError(f"q must have shape [B,1,Hq,D], got {tuple(q.shape)}")
    B, _, Hq, D = q.shape
    cache_B, MAX_S, Hkv, D_cache = _cache_dims(qkv_cache)
    if B != cache_B:
        raise ValueError(f"batch mismatch: q batch={B}, cache batch={cache_B}")
    if D != D_cache:
        raise ValueError(f"head_dim mismatch: q D={D}, cache D={D_cache}")
    validate_gqa_heads(Hq, Hkv)
    lengths_arr = normalize_positions(lengths if lengths is not None else MAX_S, B, MAX_S + 1, device=q.device)
    lengths_arr = torch.clamp(lengths_arr, max=MAX_S)
    return lengths_arr, B, MAX_S, Hq, Hkv, D


_identity_tables: dict = {}


def _identity_table(B: int, blocks: int, device) -> torch.Tensor:
    key = (B, blocks, device)
    table = _identity_tables.get(key)
    if table is None:
        table = torch.arange(B * blocks, dtype=torch.int32, device=device).reshape(B, blocks)
        _identity_tables[key] = table
    return table


def as_paged_view(qkv_cache: QuantizedKVCache, lengths_arr: torch.Tensor) -> PagedQuantizedKVCache:
    """The same buffers as a paged cache with an identity block table (no copy)."""
    B, MAX_S, Hkv, D = _cache_dims(qkv_cache)
    page = _FAST_PAGE if MAX_S % _FAST_PAGE == 0 else MAX_S
    blocks = MAX_S // page
    kq, vq = _cabi.contiguous(qkv_cache.k_q), _cabi.contiguous(qkv_cache.v_q)
    ks, vs = _cabi.contiguous(qkv_cache.k_scales), _cabi.contiguous(qkv_cache.v_scales)
    return PagedQuantizedKVCache(
        k_pages_q=kq.reshape(B * blocks, page, Hkv, kq.shape[-1]), v_pages_q=vq.reshape(B * blocks, page, Hkv, vq.shape[-1]),
        k_scales=ks.reshape(B * blocks, page, Hkv, ks.shape[-1]), v_scales=vs.reshape(B * blocks, page, Hkv, vs.shape[-1]),
        block_table=_identity_table(B, blocks, kq.device), lengths=lengths_arr, bits=qkv_cache.bits, page_size=page,
        group_size=qkv_cache.group_size, original_page_shape=(B * blocks, page, Hkv, D),
    )


def reference_quantized_kv_gqa_decode_attention(q, qkv_cache, lengths=None, *, scale=None):
    _cabi.reference_unavailable("reference_quantized_kv_gqa_decode_attention")


def quantized_kv_gqa_decode_attention(q, qkv_cache: QuantizedKVCache, lengths=None, *, scale=None,
                                      backend: str = "reference"):
    """q [B,1,Hq,D] -> [B,1,Hq,D] over the first ``lengths[b]`` tokens of every sequence (all MAX_S when
    ``lengths`` is None).  Backends: ``"cuda"`` (picks the kernel from ``qkv_cache.bits``), or the reference's
    ``"metal_q8"`` / ``"metal_q4"`` with their bits precondition; the default ``"reference"`` names the
    pure-MLX path and raises here (ops/quantized_kv_cache_ops.py:506-536).  A sequence of length 0 gives
    zeros (the reference's masked softmax would average all MAX_S positions there)."""
    lengths_arr, B, MAX_S, Hq, Hkv, D = _validate_quantized_decode_inputs(q, qkv_cache, lengths)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    name = backend.lower()
    if name == "reference":
        _cabi.reference_unavailable("quantized_kv_gqa_decode_attention")
    if name == "metal_q8":
        if qkv_cache.bits != 8:
            raise ValueError(f"metal_q8 backend requires bits=8, got bits={qkv_cache.bits}")
    elif name == "metal_q4":
        if qkv_cache.bits != 4:
            raise ValueError(f"metal_q4 backend requires bits=4, got bits={qkv_cache.bits}")
    elif name not in ("cuda", "auto"):
        raise ValueError(f"backend must be one of 'reference', 'metal_q8', 'metal_q4', 'cuda', got {name!r}")
    if D > _MAX_HEAD_DIM:
        raise ValueError(f"{name} backend supports D <= {_MAX_HEAD_DIM}, got D={D}")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"q dtype must be float16 or bfloat16, got {q.dtype}")
    _cabi.require_cuda(q, qkv_cache.k_q, qkv_cache.v_q, qkv_cache.k_scales, qkv_cache.v_scales)
    out = paged_attention_launch(q.reshape(B, Hq, D), as_paged_view(qkv_cache, lengths_arr), scale)
    return out.reshape(B, 1, Hq, D)


# ---------------------------------------------------------------------------------------------
# sliding-window (+ sink) decode over a quantised cache
# ---------------------------------------------------------------------------------------------
def reference_quantized_kv_sparse_gqa_decode_attention(q, qkv_cache, lengths, pattern, *, scale=None):
    _cabi.reference_unavailable("reference_quantized_kv_sparse_gqa_decode_attention")


def quantized_kv_sparse_gqa_decode_attention(q, qkv_cache, lengths, pattern, *, scale=None, backend: str = "reference"):
    """The reference offers this with ``backend="reference"`` only; its Metal backends raise NotImplementedError
    (ops/quantized_kv_cache_ops.py:586-603), and so do the Metal names here.  ``backend="cuda"`` runs the dense,
    sliding_window and sliding_window_sink patterns on the split-KV kernels, which skip the pages outside the
    window, and block_sparse on the same kernels over the attended pages."""
    if not isinstance(pattern, SparseAttentionPattern):
        raise TypeError("pattern must be a SparseAttentionPattern")
    name = backend.lower()
    if name == "reference":
        _cabi.reference_unavailable("quantized_kv_sparse_gqa_decode_attention")
    if name not in ("cuda", "auto"):
        raise NotImplementedError(
            "Metal sparse+quantized backend is not implemented yet. "
            "Use backend='reference' or see sparse+gqa decode attention for fp16."
        )
    block_sparse = pattern.validate().pattern == "block_sparse"
    sink_tokens, window_size = (0, 0) if block_sparse else decode_window(pattern)
    lengths_arr, B, MAX_S, Hq, Hkv, D = _validate_quantized_decode_inputs(q, qkv_cache, lengths)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if D > _MAX_HEAD_DIM:
        raise ValueError(f"{name} backend supports D <= {_MAX_HEAD_DIM}, got D={D}")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"q dtype must be float16 or bfloat16, got {q.dtype}")
    _cabi.require_cuda(q, qkv_cache.k_q, qkv_cache.v_q, qkv_cache.k_scales, qkv_cache.v_scales)
    if block_sparse:
        mask, block_size = decode_block_mask(pattern, q.device)
        out = paged_attention_launch(q.reshape(B, Hq, D), as_paged_view(qkv_cache, lengths_arr), scale,
                                     block_mask=mask, block_size=block_size)
    else:
        out = paged_attention_launch(q.reshape(B, Hq, D), as_paged_view(qkv_cache, lengths_arr), scale,
                                     sink_tokens=sink_tokens, window_size=window_size)
    return out.reshape(B, 1, Hq, D)
