"""Oracle (test infrastructure): paged q4/q8 KV pages and GQA decode attention.

Vectorised restatement of ops/paged_quantized_kv_ops.py.  The reference loops
in Python over every (page, slot, head, group); the arithmetic per group is
reproduced here on whole tensors.  The reference attention only runs when all
lengths equal MAX_BLOCKS*PAGE_SIZE (it stacks per-sequence gathers of unequal
length, ops/paged_quantized_kv_ops.py:493-510); the ragged rule used here is
the one its Metal kernels define (valid tokens are [0, lengths[b]), entries of
the block table below zero are skipped,
kernels/q4_paged_gqa_decode_attention.metal:37-58).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch

from .paged_kv_ops import validate_gqa_heads
from .quant_ops import pack_q4, unpack_q4_reference


@dataclass
class OraclePagedKV:
    """Field-for-field twin of PagedQuantizedKVCache (ops/paged_quantized_kv_ops.py:69-83)."""
    k_pages_q: Any
    v_pages_q: Any
    k_scales: Any
    v_scales: Any
    block_table: Any
    lengths: Any
    k_zeros: Any | None = None
    v_zeros: Any | None = None
    bits: int = 8
    page_size: int = 16
    group_size: int = 32
    original_page_shape: tuple[int, ...] | None = None
    metadata: dict[str, Any] = field(default_factory=dict)


def _quantize_groups_symmetric(values_f32: torch.Tensor, group_size: int, limit: int, offset: int,
                               eps: float = 1e-8):
    """_quantize_group_symmetric_8/_4 (ops/paged_quantized_kv_ops.py:146-153, 168-175) applied to
    every group of the last axis at once.  Zero padding of a short last group cannot change
    max|v| and is sliced off again."""
    D = values_f32.shape[-1]
    groups = (D + group_size - 1) // group_size
    pad = groups * group_size - D
    v = torch.nn.functional.pad(values_f32, (0, pad)) if pad else values_f32
    v = v.reshape(*values_f32.shape[:-1], groups, group_size)
    max_abs = v.abs().amax(dim=-1, keepdim=True).clamp_min(eps)
    scale = max_abs / float(limit)
    q_signed = torch.round(v / scale).clamp(-limit, limit)          # mx.round == rint
    q_unsigned = (q_signed + offset).to(torch.uint8)
    codes = q_unsigned.reshape(*values_f32.shape[:-1], groups * group_size)[..., :D]
    return codes.contiguous(), scale.squeeze(-1).to(torch.float16)


def quantize_kv_pages(K_pages, V_pages, block_table, lengths, *, bits=8, page_size=16, group_size=32):
    """ops/paged_quantized_kv_ops.py:194-292 (symmetric, scale only, fp16 scales)."""
    if bits not in (4, 8):
        raise ValueError(f"bits must be 4 or 8, got {bits}")
    if K_pages.shape != V_pages.shape:
        raise ValueError(f"K_pages and V_pages must match, got {tuple(K_pages.shape)} != {tuple(V_pages.shape)}")
    if K_pages.ndim != 4:
        raise ValueError(f"K_pages must be 4-D [NUM_PAGES,PAGE_SIZE,Hkv,D], got {tuple(K_pages.shape)}")
    NUM_PAGES, PAGE_SIZE, Hkv, D = K_pages.shape
    limit, offset = (127, 128) if bits == 8 else (7, 8)
    out = {}
    for name, pages in (("k", K_pages), ("v", V_pages)):
        codes, scales = _quantize_groups_symmetric(pages.to(torch.float32), group_size, limit, offset)
        if bits == 4:
            codes = pack_q4(codes.reshape(-1, D)).reshape(NUM_PAGES, PAGE_SIZE, Hkv, (D + 1) // 2)
        out[name] = (codes, scales)
    return OraclePagedKV(
        k_pages_q=out["k"][0], v_pages_q=out["v"][0], k_scales=out["k"][1], v_scales=out["v"][1],
        block_table=block_table, lengths=lengths, bits=bits, page_size=page_size, group_size=group_size,
        original_page_shape=tuple(K_pages.shape),
    )


def _dequant_pages(codes_q, scales, bits, group_size, shape):
    """_dequant_group_symmetric_8/_4 + cast (ops/paged_quantized_kv_ops.py:156-165, 178-186, 303-339):
    (code - 128|8) * |scale| in fp32, then fp16."""
    NUM_PAGES, PAGE_SIZE, Hkv, D = shape
    if bits == 4:
        codes = unpack_q4_reference(codes_q.reshape(-1, codes_q.shape[-1]), K=D).reshape(NUM_PAGES, PAGE_SIZE, Hkv, D)
        signed = codes.to(torch.float32) - 8.0
    else:
        signed = codes_q.to(torch.float32) - 128.0
    scale_expanded = scales.to(torch.float32).repeat_interleave(group_size, dim=-1)[..., :D]
    return (signed * scale_expanded.abs()).to(torch.float16)


def dequantize_kv_pages(cache):
    """ops/paged_quantized_kv_ops.py:295-341."""
    if cache.original_page_shape is None:
        raise ValueError("original_page_shape is required for dequantization")
    shape = tuple(cache.original_page_shape)
    K = _dequant_pages(cache.k_pages_q, cache.k_scales, cache.bits, cache.group_size, shape)
    V = _dequant_pages(cache.v_pages_q, cache.v_scales, cache.bits, cache.group_size, shape)
    return K, V


def contiguous_kv_to_pages(K_cache, V_cache, lengths, *, page_size):
    """Identity block table, unassigned entries -1 (ops/paged_quantized_kv_ops.py:375-403)."""
    if K_cache.ndim != 4 or V_cache.ndim != 4:
        raise ValueError(f"K_cache/V_cache must be 4-D [B,MAX_S,Hkv,D], got {tuple(K_cache.shape)}, {tuple(V_cache.shape)}")
    B, MAX_S, Hkv, D = K_cache.shape
    max_blocks = (MAX_S + page_size - 1) // page_size
    K_pages = torch.zeros((B * max_blocks, page_size, Hkv, D), dtype=K_cache.dtype)
    V_pages = torch.zeros((B * max_blocks, page_size, Hkv, D), dtype=V_cache.dtype)
    block_table = torch.full((B, max_blocks), -1, dtype=torch.int32)
    length_list = [int(v) for v in (lengths.tolist() if hasattr(lengths, "tolist") else lengths)]
    for b, valid in enumerate(length_list):
        for pos in range(valid):
            page_id = b * max_blocks + pos // page_size
            K_pages[page_id, pos % page_size] = K_cache[b, pos]
            V_pages[page_id, pos % page_size] = V_cache[b, pos]
            block_table[b, pos // page_size] = page_id
    return K_pages, V_pages, block_table, torch.tensor(length_list, dtype=torch.int32)


def pages_to_contiguous_kv(K_pages, V_pages, block_table, lengths, *, max_seq_len=None):
    """ops/paged_quantized_kv_ops.py:406-432."""
    B, MAX_BLOCKS = block_table.shape
    _, PAGE_SIZE, Hkv, D = K_pages.shape
    if max_seq_len is None:
        max_seq_len = MAX_BLOCKS * PAGE_SIZE
    K_cache = torch.zeros((B, max_seq_len, Hkv, D), dtype=K_pages.dtype)
    V_cache = torch.zeros((B, max_seq_len, Hkv, D), dtype=V_pages.dtype)
    for b in range(B):
        for pos in range(int(lengths[b])):
            page_id = int(block_table[b, pos // PAGE_SIZE])
            if page_id < 0:
                continue
            K_cache[b, pos] = K_pages[page_id, pos % PAGE_SIZE]
            V_cache[b, pos] = V_pages[page_id, pos % PAGE_SIZE]
    return K_cache, V_cache


def reference_paged_quantized_kv_gqa_decode_attention(q, cache, *, scale=None, window=None, keep_fn=None):
    """softmax(scale * q K^T) V over the valid tokens of every sequence, K and V dequantised
    and rounded to fp16 first, fp32 math, result cast to q.dtype
    (ops/paged_quantized_kv_ops.py:469-515, generalised to ragged lengths).

    ``window=(sink, recent)`` keeps only the first ``sink`` and last ``recent`` valid positions,
    the mask shape used by the reference's sparse scaffold
    (ops/paged_quantized_kv_ops.py:669-714); ``None`` means dense.  ``keep_fn(L)`` -> bool [L] is any other decode
    row of that scaffold's mask (block_sparse).  The scaffold masks scores to -1e9; dropping the masked keys is the
    same softmax whenever one key is visible, and a row that hides every key gives zeros here.
    """
    if q.ndim != 4 or q.shape[1] != 1:
        raise ValueError(f"q must have shape [B,1,Hq,D], got {tuple(q.shape)}")
    B, _, Hq, D = q.shape
    if cache.original_page_shape is None:
        raise ValueError("original_page_shape is required for decode attention")
    _, P, Hkv, D_cache = cache.original_page_shape
    if B != cache.block_table.shape[0]:
        raise ValueError(f"batch mismatch: q batch={B}, cache batch={cache.block_table.shape[0]}")
    if D != D_cache:
        raise ValueError(f"head_dim mismatch: q D={D}, cache D={D_cache}")
    validate_gqa_heads(Hq, Hkv)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    MAX_BLOCKS = cache.block_table.shape[1]
    lengths = torch.minimum(cache.lengths.reshape(B).to(torch.int64), torch.tensor(MAX_BLOCKS * P))

    K_deq, V_deq = dequantize_kv_pages(cache)
    Kf, Vf, qf = K_deq.to(torch.float32), V_deq.to(torch.float32), q.to(torch.float32)
    group = Hq // Hkv
    out = torch.zeros((B, 1, Hq, D), dtype=torch.float32)
    bt = cache.block_table.to(torch.int64)
    for b in range(B):
        L = int(lengths[b])
        if L <= 0:
            continue
        pos = torch.arange(L)
        pages = bt[b, pos // P]
        keep = pages >= 0
        if window is not None:
            sink, recent = window
            keep &= (pos < sink) | (pos >= L - recent)
        if keep_fn is not None:
            keep &= keep_fn(L)
        pos, pages = pos[keep], pages[keep]
        if pos.numel() == 0:
            continue
        Kb = Kf[pages, pos % P]            # [L', Hkv, D]
        Vb = Vf[pages, pos % P]
        qb = qf[b, 0].reshape(Hkv, group, D)
        scores = torch.einsum("hgd,lhd->hgl", qb, Kb) * float(scale)
        probs = torch.softmax(scores, dim=-1)
        out[b, 0] = torch.einsum("hgl,lhd->hgd", probs, Vb).reshape(Hq, D)
    return out.to(q.dtype)
