"""GQA head helpers (reference ops/gqa_ops.py:42-66)."""
from __future__ import annotations


def validate_gqa_heads(num_attention_heads: int, num_key_value_heads: int) -> None:
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


def gqa_group_size(num_attention_heads: int, num_key_value_heads: int) -> int:
    validate_gqa_heads(num_attention_heads, num_key_value_heads)
    return num_attention_heads // num_key_value_heads


def q_head_to_kv_head(q_head: int, num_attention_heads: int, num_key_value_heads: int) -> int:
    group = gqa_group_size(num_attention_heads, num_key_value_heads)
    if q_head < 0 or q_head >= num_attention_heads:
        raise ValueError(f"q_head must be in [0, {num_attention_heads}), got {q_head}")
    return q_head // group
