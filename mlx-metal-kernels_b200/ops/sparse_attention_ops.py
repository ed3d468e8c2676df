"""Sparse attention patterns as far as the quantized decode path uses them.

Mirrors the pattern dataclass of ops/sparse_attention_ops.py:20-47 of the reference.  For single-token
decode the query sits at position L - 1 of a sequence of L tokens, so a sliding-window pattern reduces to a
(sink_tokens, window_size) pair: the row of build_sparse_attention_mask
(ops/sparse_attention_ops.py:85-105) that a decode step sees is ``j < sink_tokens or j >= L - window_size``;
a block_sparse pattern reduces to row (L - 1) // block_size of its block mask
(ops/sparse_attention_ops.py:98-107).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass
class SparseAttentionPattern:
    pattern: str
    window_size: int | None = None
    sink_tokens: int = 0
    block_size: int | None = None
    block_mask: Any | None = None
    causal: bool = True

    def validate(self) -> "SparseAttentionPattern":
        if self.pattern not in ("dense", "sliding_window", "sliding_window_sink", "block_sparse"):
            raise ValueError(
                "pattern must be one of 'dense', 'sliding_window', 'sliding_window_sink', 'block_sparse'"
            )
        if self.sink_tokens < 0:
            raise ValueError(f"sink_tokens must be >= 0, got {self.sink_tokens}")
        if self.pattern == "sliding_window":
            if self.window_size is None or self.window_size <= 0:
                raise ValueError("sliding_window requires window_size > 0")
        if self.pattern == "sliding_window_sink":
            if self.window_size is None or self.window_size <= 0:
                raise ValueError("sliding_window_sink requires window_size > 0")
        if self.pattern == "block_sparse":
            if self.block_size is None or self.block_size <= 0:
                raise ValueError("block_sparse requires block_size > 0")
            if self.block_mask is None:
                raise ValueError("block_sparse requires block_mask")
        return self


def decode_window(pattern: SparseAttentionPattern) -> tuple[int, int]:
    """(sink_tokens, window_size) of the decode row of ``pattern``; (0, 0) means dense.
    ``sliding_window`` ignores ``sink_tokens``, as the reference's mask builder does."""
    if not isinstance(pattern, SparseAttentionPattern):
        raise TypeError("pattern must be a SparseAttentionPattern")
    pattern = pattern.validate()
    if pattern.pattern == "dense":
        return 0, 0
    if pattern.pattern == "sliding_window":
        return 0, int(pattern.window_size)
    if pattern.pattern == "sliding_window_sink":
        return int(pattern.sink_tokens), int(pattern.window_size)
    raise ValueError("block_sparse has no (sink, window) form; use decode_block_mask")


def decode_block_mask(pattern: SparseAttentionPattern, device):
    """(block_mask uint8 [n_qblocks, n_kblocks] on ``device``, block_size) of a block_sparse pattern."""
    import torch
    pattern = pattern.validate()
    if pattern.pattern != "block_sparse":
        raise ValueError("decode_block_mask needs a block_sparse pattern")
    mask = pattern.block_mask
    if hasattr(mask, "tolist") and not isinstance(mask, torch.Tensor):
        mask = mask.tolist()
    mask = torch.as_tensor(mask)
    if mask.ndim != 2 or mask.shape[0] == 0 or mask.shape[1] == 0:
        raise ValueError(f"block_mask must be 2-D [q_blocks, k_blocks], got {tuple(mask.shape)}")
    return (mask != 0).to(device=device, dtype=torch.uint8).contiguous(), int(pattern.block_size)
