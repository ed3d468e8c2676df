"""Oracle (test infrastructure): block-table gather, GQA head helpers and decode attention over an unquantised
paged KV cache.

The attention restates reference_paged_decode_attention (ops/paged_kv_ops.py:258-304) and
reference_paged_gqa_decode_attention (ops/gqa_ops.py:307-340 with reference_gqa_decode_attention,
ops/gqa_ops.py:262-304): gather the pages of every sequence through the block table, fp32 scores scale * q . k,
positions >= length masked out, softmax, fp32 weighted sum of V, cast to q's dtype.  That part is not pinned by a
reference run (the reference functions are MLX-only); it is the same masked softmax the pinned quantised
attention bodies compute, on unquantised rows.
"""
from __future__ import annotations

import math

import torch


def validate_gqa_heads(num_attention_heads: int, num_key_value_heads: int) -> None:
    """ops/gqa_ops.py:42-54."""
    if num_key_value_heads < 1:
        raise ValueError(f"num_key_value_heads must be >= 1, got {num_key_value_heads}")
    if num_attention_heads < num_key_value_heads:
        raise ValueError(
            "num_attention_heads must be >= num_key_value_heads, "
            f"got {num_attention_heads}, {num_key_value_heads}"
        )
    if num_attention_heads % num_key_value_heads != 0:
        raise ValueError(
            "num_attention_heads must be divisible by num_key_value_heads, "
            f"got {num_attention_heads}, {num_key_value_heads}"
        )


def q_head_to_kv_head(q_head: int, num_attention_heads: int, num_key_value_heads: int) -> int:
    """ops/gqa_ops.py:62-66."""
    validate_gqa_heads(num_attention_heads, num_key_value_heads)
    if q_head < 0 or q_head >= num_attention_heads:
        raise ValueError(f"q_head must be in [0, {num_attention_heads}), got {q_head}")
    return q_head // (num_attention_heads // num_key_value_heads)


def normalize_positions(positions, B: int, MAX_S: int) -> torch.Tensor:
    """Scalar or [B] positions -> int32 [B], range-checked (ops/kv_cache_ops.py:37-61)."""
    if isinstance(positions, int):
        pos = torch.full((B,), positions, dtype=torch.int32)
    else:
        pos_arr = torch.as_tensor(positions).to(torch.int32).cpu()
        if pos_arr.ndim == 0:
            pos = torch.full((B,), int(pos_arr.item()), dtype=torch.int32)
        elif pos_arr.ndim == 1 and pos_arr.shape[0] == B:
            pos = pos_arr
        else:
            raise ValueError(f"positions must be scalar or shape [B], got {tuple(pos_arr.shape)}")
    for p in pos.tolist():
        if p < 0 or p >= MAX_S:
            raise ValueError(f"positions must be in [0, {MAX_S}), got {p}")
    return pos


def reference_block_table_lookup(block_table: torch.Tensor, positions, PAGE_SIZE: int):
    """page_ids[b] = block_table[b, pos[b] // P], offsets[b] = pos[b] % P
    (ops/paged_kv_ops.py:138-152)."""
    if PAGE_SIZE <= 0:
        raise ValueError("PAGE_SIZE must be positive")
    if block_table.ndim != 2:
        raise ValueError(f"block_table must be 2-D [B,MAX_BLOCKS], got {tuple(block_table.shape)}")
    B, MAX_BLOCKS = block_table.shape
    pos = normalize_positions(positions, B, MAX_BLOCKS * PAGE_SIZE)
    block_ids = (pos // PAGE_SIZE).to(torch.int64)
    offsets = pos % PAGE_SIZE
    page_ids = block_table.cpu()[torch.arange(B), block_ids]
    return page_ids.to(torch.int32), offsets.to(torch.int32)


def reference_paged_gqa_decode_attention(q, K_pages, V_pages, block_table, lengths=None, scale=None):
    """q [B,1,Hq,D], pages [NUM_PAGES,PAGE_SIZE,Hkv,D], block_table [B,MAX_BLOCKS], lengths [B] -> [B,1,Hq,D]."""
    if K_pages.ndim != 4 or V_pages.ndim != 4 or K_pages.shape != V_pages.shape:
        raise ValueError("K_pages and V_pages must match [NUM_PAGES,PAGE_SIZE,Hkv,D]")
    B, MAX_BLOCKS = block_table.shape
    _, P, Hkv, D = K_pages.shape
    Hq = q.shape[2]
    if Hq % Hkv:
        raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
    group = Hq // Hkv
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if lengths is None:
        lengths = torch.full((B,), MAX_BLOCKS * P, dtype=torch.int64)
    lengths = torch.as_tensor(lengths).reshape(-1).to(torch.int64).expand(B).clamp(max=MAX_BLOCKS * P)
    out = torch.zeros((B, 1, Hq, D), dtype=torch.float32)
    bt = block_table.to(torch.int64)
    for b in range(B):
        L = int(lengths[b])
        if L <= 0:
            continue
        pos = torch.arange(L)
        pages = bt[b, pos // P]
        keep = pages >= 0
        pos, pages = pos[keep], pages[keep]
        if pos.numel() == 0:
            continue
        Kb = K_pages[pages, pos % P].to(torch.float32)          # [L, Hkv, D]
        Vb = V_pages[pages, pos % P].to(torch.float32)
        qb = q[b, 0].to(torch.float32).reshape(Hkv, group, D)
        scores = torch.einsum("hgd,lhd->hgl", qb, Kb) * float(scale)
        probs = torch.softmax(scores, dim=-1)
        out[b, 0] = torch.einsum("hgl,lhd->hgd", probs, Vb).reshape(Hq, D)
    return out.to(q.dtype)


def reference_paged_decode_attention(q, K_pages, V_pages, block_table, lengths, *, scale=None):
    """The H == Hkv form (ops/paged_kv_ops.py:258-304)."""
    if q.shape[2] != K_pages.shape[2]:
        raise ValueError("q must have shape [B,1,H,D] with the cache's head count")
    return reference_paged_gqa_decode_attention(q, K_pages, V_pages, block_table, lengths, scale=scale)
