"""Block-table gather (reference ops/paged_kv_ops.py:99-182, ops/kv_cache_ops.py:37-61)."""
from __future__ import annotations

import math

import torch

from . import _cabi


def make_identity_block_table(B: int, MAX_S: int, PAGE_SIZE: int, device=None) -> torch.Tensor:
    if B <= 0 or MAX_S <= 0 or PAGE_SIZE <= 0:
        raise ValueError(f"B, MAX_S, and PAGE_SIZE must be positive, got {B}, {MAX_S}, {PAGE_SIZE}")
    max_blocks = math.ceil(MAX_S / PAGE_SIZE)
    base = torch.arange(B, dtype=torch.int32, device=device).reshape(B, 1) * max_blocks
    return base + torch.arange(max_blocks, dtype=torch.int32, device=device).reshape(1, max_blocks)


def allocate_paged_kv_cache(B: int, MAX_S: int, H: int, D: int, PAGE_SIZE: int, dtype, device=None):
    if dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"dtype must be float16 or bfloat16, got {dtype}")
    block_table = make_identity_block_table(B, MAX_S, PAGE_SIZE, device=device)
    num_pages = B * math.ceil(MAX_S / PAGE_SIZE)
    K_pages = torch.zeros((num_pages, PAGE_SIZE, H, D), dtype=dtype, device=device)
    V_pages = torch.zeros((num_pages, PAGE_SIZE, H, D), dtype=dtype, device=device)
    return K_pages, V_pages, block_table


def normalize_positions(positions, B: int, MAX_S: int, device=None) -> torch.Tensor:
    """Scalar or [B] positions -> int32 [B]; values outside [0, MAX_S) raise, as in the reference.
    The range check reads the values on the host, like the reference's ``tolist()``."""
    if isinstance(positions, int):
        pos = torch.full((B,), positions, dtype=torch.int32, device=device)
    else:
        pos_arr = positions if isinstance(positions, torch.Tensor) else torch.as_tensor(positions)
        if pos_arr.ndim == 0:
            pos = torch.full((B,), int(pos_arr.item()), dtype=torch.int32, device=device)
        elif pos_arr.ndim == 1 and pos_arr.shape[0] == B:
            pos = pos_arr.to(device=device, dtype=torch.int32)
        else:
            raise ValueError(f"positions must be scalar or shape [B], got {tuple(pos_arr.shape)}")
    for p in pos.tolist():
        if p < 0 or p >= MAX_S:
            raise ValueError(f"positions must be in [0, {MAX_S}), got {p}")
    return pos


def reference_block_table_lookup(block_table, positions, PAGE_SIZE: int):
    _cabi.reference_unavailable("reference_block_table_lookup")


def block_table_lookup(block_table, positions, PAGE_SIZE: int, *, backend: str = "auto"):
    """(page_ids, offsets), both int32 [B]: page_ids[b] = block_table[b, pos[b] // PAGE_SIZE],
    offsets[b] = pos[b] % PAGE_SIZE."""
    if PAGE_SIZE <= 0:
        raise ValueError("PAGE_SIZE must be positive")
    if block_table.ndim != 2:
        raise ValueError(f"block_table must be 2-D [B,MAX_BLOCKS], got {tuple(block_table.shape)}")
    B, MAX_BLOCKS = block_table.shape
    pos = normalize_positions(positions, B, MAX_BLOCKS * PAGE_SIZE, device=block_table.device)
    name = backend.lower()
    if _cabi.safe_mode_enabled() or name == "reference":
        _cabi.reference_unavailable("block_table_lookup")
    if name not in ("auto", "metal", "cuda"):
        raise ValueError("backend must be one of 'reference', 'metal', 'auto', 'cuda'")
    _cabi.require_cuda(block_table, pos)
    bt = _cabi.contiguous(block_table.to(torch.int32))
    pos = _cabi.contiguous(pos)
    page_ids = torch.empty((B,), dtype=torch.int32, device=bt.device)
    offsets = torch.empty((B,), dtype=torch.int32, device=bt.device)
    _cabi.check(
        _cabi.load().b200q_block_table_lookup(bt.data_ptr(), pos.data_ptr(), page_ids.data_ptr(), offsets.data_ptr(),
                                              B, MAX_BLOCKS, PAGE_SIZE, _cabi.stream()),
        "b200q_block_table_lookup",
    )
    return page_ids, offsets
