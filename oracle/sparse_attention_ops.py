"""Oracle (test infrastructure): the reference's sparse attention mask rule.

Restates build_sparse_attention_mask (ops/sparse_attention_ops.py:73-112) for the patterns the
quantized decode path uses, as plain Python loops over positions (test sizes only).
"""
from __future__ import annotations

import torch


def build_sparse_attention_mask(Sq: int, Sk: int, pattern: str, *, window_size=None, sink_tokens: int = 0,
                                causal: bool = True, start_position: int = 0, block_size=None,
                                block_mask=None) -> torch.Tensor:
    """bool [Sq, Sk]: query i sits at absolute position start_position + i.
    dense: j <= q (causal) or everything; sliding_window: max(0, q - W + 1) <= j <= q;
    sliding_window_sink: additionally j < sink_tokens (and j <= q);
    block_sparse: block_mask[q // block_size][j // block_size] (and j <= q when causal)."""
    if pattern not in ("dense", "sliding_window", "sliding_window_sink", "block_sparse"):
        raise ValueError("pattern must be one of 'dense', 'sliding_window', 'sliding_window_sink', 'block_sparse'")
    if pattern == "block_sparse" and hasattr(block_mask, "tolist"):
        block_mask = block_mask.tolist()
    if Sq <= 0 or Sk <= 0:
        raise ValueError(f"Sq and Sk must be positive, got {Sq}, {Sk}")
    if start_position < 0:
        raise ValueError(f"start_position must be >= 0, got {start_position}")
    rows = []
    for i in range(Sq):
        q_abs = start_position + i
        row = []
        for j in range(Sk):
            if pattern == "dense":
                visible = True if not causal else (j <= q_abs)
            elif pattern == "block_sparse":
                visible = bool(block_mask[q_abs // int(block_size)][j // int(block_size)])
                if causal:
                    visible = visible and (j <= q_abs)
            else:
                local_start = max(0, q_abs - int(window_size) + 1)
                visible = local_start <= j <= q_abs
                if pattern == "sliding_window_sink":
                    visible = visible or ((j < sink_tokens) and (j <= q_abs))
            row.append(bool(visible))
        rows.append(row)
    return torch.tensor(rows, dtype=torch.bool)


def decode_row(valid_len: int, pattern: str, *, window_size=None, sink_tokens: int = 0, block_size=None,
               block_mask=None) -> torch.Tensor:
    """The mask row of a decode step over ``valid_len`` tokens, as the reference's sparse scaffolds build it
    (ops/paged_quantized_kv_ops.py:693, ops/quantized_kv_cache_ops.py:563): one query at position valid_len - 1."""
    return build_sparse_attention_mask(1, valid_len, pattern, window_size=window_size, sink_tokens=sink_tokens,
                                       start_position=valid_len - 1, block_size=block_size, block_mask=block_mask)[0]
