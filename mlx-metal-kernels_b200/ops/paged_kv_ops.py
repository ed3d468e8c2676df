"""Block-table gather (reference ops/paged_kv_ops.py:99-182, ops/kv_cache_ops.py:37-61) and decode attention over
an unquantised paged cache (ops/paged_kv_ops.py:258-360, ops/gqa_ops.py:307-340)."""
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


def _validate_page_tensors(K_pages, V_pages, block_table):
    if K_pages.ndim != 4 or V_pages.ndim != 4:
        raise ValueError(f"K_pages and V_pages must be [NUM_PAGES,PAGE_SIZE,H,D], got {tuple(K_pages.shape)}, {tuple(V_pages.shape)}")
    if K_pages.shape != V_pages.shape:
        raise ValueError(f"K_pages and V_pages must have identical shapes, got {tuple(K_pages.shape)}, {tuple(V_pages.shape)}")
    if block_table.ndim != 2:
        raise ValueError(f"block_table must be [B,MAX_BLOCKS], got {tuple(block_table.shape)}")
    NUM_PAGES, PAGE_SIZE, H, D = K_pages.shape
    B, MAX_BLOCKS = block_table.shape
    return NUM_PAGES, PAGE_SIZE, H, D, B, MAX_BLOCKS


_workspaces: dict = {}


def paged_fp16_attention_launch(q3d, K_pages, V_pages, block_table, lengths, scale):
    """q3d [B,Hq,D], pages [NUM_PAGES,PAGE_SIZE,Hkv,D] in q's dtype, lengths int32 [B] -> [B,Hq,D]."""
    B, Hq, D = q3d.shape
    NUM_PAGES, PAGE_SIZE, Hkv, _ = K_pages.shape
    MAX_BLOCKS = block_table.shape[1]
    lib = _cabi.load()
    q3d = _cabi.contiguous(q3d)
    K_pages, V_pages = _cabi.contiguous(K_pages.to(q3d.dtype)), _cabi.contiguous(V_pages.to(q3d.dtype))
    bt = _cabi.contiguous(block_table.to(torch.int32))
    ln = _cabi.contiguous(lengths.reshape(B).to(torch.int32))
    out = torch.empty_like(q3d)
    nbytes = lib.b200q_paged_fp16_gqa_workspace_bytes(B, Hq, Hkv, MAX_BLOCKS)
    key = (q3d.device, torch.cuda.current_stream(q3d.device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < max(nbytes, 16):
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q3d.device)
        _workspaces[key] = ws
    _cabi.check(lib.b200q_paged_fp16_gqa_decode(q3d.data_ptr(), K_pages.data_ptr(), V_pages.data_ptr(), bt.data_ptr(),
                                                ln.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), B, Hq, Hkv, D,
                                                PAGE_SIZE, NUM_PAGES, MAX_BLOCKS, float(scale),
                                                _cabi.dtype_code(q3d.dtype), _cabi.stream()),
                "b200q_paged_fp16_gqa_decode")
    return out


def _lengths_for_decode(lengths, B: int, capacity: int, device):
    """Scalar / [B] / None lengths -> int32 [B] in [0, capacity] (checked on the host like the reference's)."""
    return normalize_positions(capacity if lengths is None else lengths, B, capacity + 1, device=device)


def reference_paged_decode_attention(q, K_pages, V_pages, block_table, lengths, *, scale=None):
    _cabi.reference_unavailable("reference_paged_decode_attention")


def paged_decode_attention(q, K_pages, V_pages, block_table, lengths, *, scale=None, backend: str = "auto"):
    """Decode attention over an fp16 / bf16 paged cache, q [B,1,H,D] with as many query as kv heads
    (ops/paged_kv_ops.py:307-360 of the reference; for Hq != Hkv see ``paged_gqa_decode_attention``).  Every Metal
    backend name selects the one CUDA kernel."""
    NUM_PAGES, PAGE_SIZE, H, D, B, MAX_BLOCKS = _validate_page_tensors(K_pages, V_pages, block_table)
    if q.ndim != 4 or tuple(q.shape) != (B, 1, H, D):
        raise ValueError(
            f"q must have shape [B,1,H,D]={B,1,H,D}, got {tuple(q.shape)}. "
            "For GQA/MQA paged decode with Hq != Hkv, use ops.gqa_ops.reference_paged_gqa_decode_attention."
        )
    if D > 128:
        raise ValueError(f"paged_decode_attention currently supports D <= 128, got {D}")
    lengths_arr = _lengths_for_decode(lengths, B, MAX_BLOCKS * PAGE_SIZE, q.device)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    name = backend.lower()
    if _cabi.safe_mode_enabled() or name == "reference":
        _cabi.reference_unavailable("paged_decode_attention")
    if name not in ("auto", "cuda", "metal", "metal_threadgroup", "metal_d64", "metal_d128"):
        raise ValueError("backend must be one of 'reference', 'metal', 'metal_threadgroup', 'metal_d64', 'metal_d128', "
                         "'auto', 'cuda'")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"q dtype must be float16 or bfloat16, got {q.dtype}")
    _cabi.require_cuda(q, K_pages, V_pages, block_table, lengths_arr)
    return paged_fp16_attention_launch(q.reshape(B, H, D), K_pages, V_pages, block_table, lengths_arr, scale).reshape(B, 1, H, D)
