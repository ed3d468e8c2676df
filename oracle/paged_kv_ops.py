"""Oracle (test infrastructure): block-table gather and GQA head helpers."""
from __future__ import annotations

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
