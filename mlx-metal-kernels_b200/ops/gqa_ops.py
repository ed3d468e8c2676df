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


def reference_paged_gqa_decode_attention(q, K_pages, V_pages, block_table, lengths=None, scale=None):
    from . import _cabi
    _cabi.reference_unavailable("reference_paged_gqa_decode_attention")


def paged_gqa_decode_attention(q, K_pages, V_pages, block_table, lengths=None, scale=None, *, backend: str = "cuda"):
    """Grouped-query decode attention over an fp16 / bf16 paged cache: q [B,1,Hq,D], pages
    [NUM_PAGES,PAGE_SIZE,Hkv,D] -> [B,1,Hq,D].  The reference has only the pure-MLX form
    (reference_paged_gqa_decode_attention, ops/gqa_ops.py:307-340); here it runs on the CUDA kernel."""
    import math

    import torch

    from . import _cabi, paged_kv_ops
    if K_pages.ndim != 4 or V_pages.ndim != 4 or K_pages.shape != V_pages.shape:
        raise ValueError(f"K_pages and V_pages must match [NUM_PAGES,PAGE_SIZE,Hkv,D], got {tuple(K_pages.shape)}, {tuple(V_pages.shape)}")
    if block_table.ndim != 2:
        raise ValueError(f"block_table must be [B,MAX_BLOCKS], got {tuple(block_table.shape)}")
    NUM_PAGES, PAGE_SIZE, Hkv, D = K_pages.shape
    B, MAX_BLOCKS = block_table.shape
    if q.ndim != 4 or q.shape[0] != B or q.shape[1] != 1 or q.shape[3] != D:
        raise ValueError(f"q must have shape [B,1,Hq,D] with B={B}, D={D}, got {tuple(q.shape)}")
    Hq = q.shape[2]
    validate_gqa_heads(Hq, Hkv)
    if D > 128:
        raise ValueError(f"paged_gqa_decode_attention supports D <= 128, got {D}")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"q dtype must be float16 or bfloat16, got {q.dtype}")
    name = backend.lower()
    if _cabi.safe_mode_enabled() or name == "reference":
        _cabi.reference_unavailable("paged_gqa_decode_attention")
    if name not in ("cuda", "auto", "metal"):
        raise ValueError("backend must be one of 'reference', 'cuda', 'auto'")
    lengths_arr = paged_kv_ops._lengths_for_decode(lengths, B, MAX_BLOCKS * PAGE_SIZE, q.device)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    _cabi.require_cuda(q, K_pages, V_pages, block_table, lengths_arr)
    out = paged_kv_ops.paged_fp16_attention_launch(q.reshape(B, Hq, D), K_pages, V_pages, block_table, lengths_arr, scale)
    return out.reshape(B, 1, Hq, D)
