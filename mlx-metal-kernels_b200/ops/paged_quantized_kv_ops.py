"""Paged quantized KV cache (q8 / q4, symmetric, fp16 scales) and its GQA decode attention.

Mirrors ops/paged_quantized_kv_ops.py of the reference: the config and cache dataclasses, page
quantise / dequantise, contiguous <-> pages helpers and the decode-attention entry point.
Layouts: codes ``[NUM_PAGES, PAGE_SIZE, Hkv, D]`` (q8) or ``[.., ceil(D/2)]`` (q4, low nibble =
even d), scales ``[NUM_PAGES, PAGE_SIZE, Hkv, ceil(D/group_size)]`` fp16, ``block_table``
``[B, MAX_BLOCKS]`` int32 (entries < 0 = unassigned), ``lengths`` ``[B]`` int32.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch

from . import _cabi
from .gqa_ops import validate_gqa_heads
from .quant_ops import dequant_codes
from .sparse_attention_ops import SparseAttentionPattern, decode_block_mask, decode_window

_MAX_HEAD_DIM = 128


def _dtype_itemsize(dtype: Any) -> int:
    return torch.empty((), dtype=dtype).element_size()


@dataclass
class PagedQuantizedKVConfig:
    bits: int = 8
    page_size: int = 16
    group_size: int = 32
    symmetric: bool = True
    with_zeros: bool = False
    scale_dtype: str = "float16"
    layout: str = "paged"

    def validate(self) -> "PagedQuantizedKVConfig":
        if self.bits not in (4, 8):
            raise ValueError(f"bits must be 4 or 8, got {self.bits}")
        if self.page_size <= 0:
            raise ValueError(f"page_size must be > 0, got {self.page_size}")
        if self.group_size <= 0:
            raise ValueError(f"group_size must be > 0, got {self.group_size}")
        if not self.symmetric:
            raise NotImplementedError("asymmetric quantization is not implemented yet")
        if self.with_zeros:
            raise NotImplementedError("zero-point quantization is not implemented yet")
        if self.layout != "paged":
            raise ValueError(f"layout must be 'paged', got {self.layout!r}")
        return self


@dataclass
class PagedQuantizedKVCache:
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

    def shapes(self) -> dict[str, tuple[int, ...] | None]:
        return {
            "k_pages_q": tuple(self.k_pages_q.shape),
            "v_pages_q": tuple(self.v_pages_q.shape),
            "k_scales": tuple(self.k_scales.shape),
            "v_scales": tuple(self.v_scales.shape),
            "block_table": tuple(self.block_table.shape),
            "lengths": tuple(self.lengths.shape),
            "original_page_shape": None if self.original_page_shape is None else tuple(self.original_page_shape),
        }

    def validate(self) -> "PagedQuantizedKVCache":
        if self.bits not in (4, 8):
            raise ValueError(f"bits must be 4 or 8, got {self.bits}")
        if self.k_pages_q.shape != self.v_pages_q.shape:
            raise ValueError(f"k_pages_q and v_pages_q shapes must match, got {tuple(self.k_pages_q.shape)} != {tuple(self.v_pages_q.shape)}")
        if self.k_scales.shape != self.v_scales.shape:
            raise ValueError(f"k_scales and v_scales shapes must match, got {tuple(self.k_scales.shape)} != {tuple(self.v_scales.shape)}")
        if self.block_table.ndim != 2:
            raise ValueError(f"block_table must be 2-D [B,MAX_BLOCKS], got {tuple(self.block_table.shape)}")
        if self.lengths.ndim != 1:
            raise ValueError(f"lengths must be 1-D [B], got {tuple(self.lengths.shape)}")
        B = self.block_table.shape[0]
        if self.lengths.shape[0] != B:
            raise ValueError(f"lengths batch {self.lengths.shape[0]} != block_table batch {B}")
        if self.original_page_shape is not None and len(self.original_page_shape) != 4:
            raise ValueError(f"original_page_shape must be 4-D [NUM_PAGES,PAGE_SIZE,Hkv,D], got {self.original_page_shape}")
        return self

    def num_pages(self) -> int:
        return self.k_pages_q.shape[0]

    def memory_bytes(self) -> int:
        total = 0
        for arr in (self.k_pages_q, self.v_pages_q, self.k_scales, self.v_scales, self.block_table, self.lengths,
                    self.k_zeros, self.v_zeros):
            if arr is not None:
                total += arr.numel() * arr.element_size()
        return total

    def compression_ratio(self, fp_bytes_per_value: int = 2) -> float | None:
        if self.original_page_shape is None:
            return None
        NUM_PAGES, PAGE_SIZE, Hkv, D = self.original_page_shape
        fp_bytes = 2 * NUM_PAGES * PAGE_SIZE * Hkv * D * fp_bytes_per_value
        q_bytes = sum(a.numel() * a.element_size() for a in (self.k_pages_q, self.v_pages_q, self.k_scales, self.v_scales))
        return None if q_bytes == 0 else fp_bytes / q_bytes


# ---------------------------------------------------------------------------------------------
# quantise / dequantise pages
# ---------------------------------------------------------------------------------------------
def _quantize_groups(values: torch.Tensor, bits: int, group_size: int):
    """Per group of the last axis: scale = max(max|v|, 1e-8) / (127|7) in fp32, code =
    clip(rint(v / scale)) + (128|8), scale stored fp16 (ops/paged_quantized_kv_ops.py:146-175).
    Returns (codes [..., D] or packed [..., ceil(D/2)], scales [..., ceil(D/group)]) from the CUDA kernel."""
    _cabi.require_cuda(values)
    if values.dtype not in (torch.float16, torch.bfloat16):
        values = values.to(torch.float16)
    values = _cabi.contiguous(values)
    D = values.shape[-1]
    rows = values.numel() // D
    groups = (D + group_size - 1) // group_size
    dp = (D + 1) // 2 if bits == 4 else D
    codes = torch.empty((*values.shape[:-1], dp), dtype=torch.uint8, device=values.device)
    scales = torch.empty((*values.shape[:-1], groups), dtype=torch.float16, device=values.device)
    _cabi.check(_cabi.load().b200q_quantize_kv(bits, values.data_ptr(), codes.data_ptr(), scales.data_ptr(), rows, D,
                                               group_size, _cabi.dtype_code(values.dtype), _cabi.stream()),
                "b200q_quantize_kv")
    return codes, scales


def quantize_kv_pages(K_pages, V_pages, block_table, lengths, config: PagedQuantizedKVConfig) -> PagedQuantizedKVCache:
    """fp16/bf16 pages [NUM_PAGES,PAGE_SIZE,Hkv,D] -> quantized cache (ops/paged_quantized_kv_ops.py:194-292)."""
    config = config.validate()
    if K_pages.shape != V_pages.shape:
        raise ValueError(f"K_pages and V_pages must match, got {tuple(K_pages.shape)} != {tuple(V_pages.shape)}")
    if K_pages.ndim != 4:
        raise ValueError(f"K_pages must be 4-D [NUM_PAGES,PAGE_SIZE,Hkv,D], got {tuple(K_pages.shape)}")
    NUM_PAGES, PAGE_SIZE, Hkv, D = K_pages.shape
    out = []
    for pages in (K_pages, V_pages):
        out.append(_quantize_groups(pages, config.bits, config.group_size))
    return PagedQuantizedKVCache(
        k_pages_q=out[0][0], v_pages_q=out[1][0], k_scales=out[0][1], v_scales=out[1][1],
        block_table=block_table, lengths=lengths, bits=config.bits, page_size=config.page_size,
        group_size=config.group_size, original_page_shape=tuple(K_pages.shape),
    )


def dequantize_kv_pages(paged_qkv: PagedQuantizedKVCache):
    """(K, V) fp16 [NUM_PAGES,PAGE_SIZE,Hkv,D] = cast((code - 128|8) * |scale|)
    (ops/paged_quantized_kv_ops.py:295-341), through the bit-exact dequant kernel."""
    paged_qkv = paged_qkv.validate()
    orig = paged_qkv.original_page_shape
    if orig is None:
        raise ValueError("original_page_shape is required for dequantization")
    NUM_PAGES, PAGE_SIZE, Hkv, D = orig
    rows = NUM_PAGES * PAGE_SIZE * Hkv
    groups = (D + paged_qkv.group_size - 1) // paged_qkv.group_size
    offset = 128.0 if paged_qkv.bits == 8 else 8.0
    outs = []
    for codes, scales in ((paged_qkv.k_pages_q, paged_qkv.k_scales), (paged_qkv.v_pages_q, paged_qkv.v_scales)):
        s = scales.reshape(rows, groups).abs()
        z = torch.full_like(s, offset)
        out = dequant_codes(paged_qkv.bits, codes.reshape(rows, codes.shape[-1]), s, z, rows, D,
                            paged_qkv.group_size, torch.float16)
        outs.append(out.reshape(NUM_PAGES, PAGE_SIZE, Hkv, D))
    return outs[0], outs[1]


def paged_quantized_kv_error(K_pages, V_pages, paged_qkv: PagedQuantizedKVCache) -> dict[str, float]:
    K_deq, V_deq = dequantize_kv_pages(paged_qkv)
    k_diff = K_pages.to(torch.float32) - K_deq.to(torch.float32)
    v_diff = V_pages.to(torch.float32) - V_deq.to(torch.float32)
    cr = paged_qkv.compression_ratio(fp_bytes_per_value=2)
    return {
        "k_max_abs_error": float(k_diff.abs().max()), "k_mean_abs_error": float(k_diff.abs().mean()),
        "k_rmse": float(k_diff.square().mean().sqrt()),
        "v_max_abs_error": float(v_diff.abs().max()), "v_mean_abs_error": float(v_diff.abs().mean()),
        "v_rmse": float(v_diff.square().mean().sqrt()),
        "compression_ratio": float(cr) if cr is not None else 0.0,
    }


# ---------------------------------------------------------------------------------------------
# contiguous <-> pages (test / demo helpers)
# ---------------------------------------------------------------------------------------------
def contiguous_kv_to_pages(K_cache, V_cache, lengths, *, page_size: int):
    """Identity block table: page = b * max_blocks + pos // page_size; unassigned entries -1."""
    if K_cache.ndim != 4 or V_cache.ndim != 4:
        raise ValueError(f"K_cache/V_cache must be 4-D [B,MAX_S,Hkv,D], got {tuple(K_cache.shape)}, {tuple(V_cache.shape)}")
    B, MAX_S, Hkv, D = K_cache.shape
    dev = K_cache.device
    max_blocks = (MAX_S + page_size - 1) // page_size
    length_list = [int(v) for v in (lengths.tolist() if hasattr(lengths, "tolist") else lengths)]
    lens = torch.tensor(length_list, dtype=torch.int32, device=dev)
    pad = max_blocks * page_size - MAX_S
    pos = torch.arange(max_blocks * page_size, device=dev)
    keep = (pos.reshape(1, -1) < lens.reshape(B, 1)).reshape(B, max_blocks * page_size, 1, 1)

    def to_pages(cache):
        c = torch.nn.functional.pad(cache, (0, 0, 0, 0, 0, pad)) if pad else cache
        c = torch.where(keep, c, torch.zeros((), dtype=cache.dtype, device=dev))
        return c.reshape(B * max_blocks, page_size, Hkv, D).contiguous()

    used = (torch.arange(max_blocks, device=dev).reshape(1, -1) * page_size) < lens.reshape(B, 1)
    ids = torch.arange(B * max_blocks, dtype=torch.int32, device=dev).reshape(B, max_blocks)
    block_table = torch.where(used, ids, torch.full_like(ids, -1))
    return to_pages(K_cache), to_pages(V_cache), block_table, lens


def pages_to_contiguous_kv(K_pages, V_pages, block_table, lengths, *, max_seq_len: int | None = None):
    B, MAX_BLOCKS = block_table.shape
    NUM_PAGES, PAGE_SIZE, Hkv, D = K_pages.shape
    dev = K_pages.device
    if max_seq_len is None:
        max_seq_len = MAX_BLOCKS * PAGE_SIZE
    pos = torch.arange(max_seq_len, device=dev)
    blk = (pos // PAGE_SIZE).clamp_max(MAX_BLOCKS - 1)
    page = block_table.to(torch.int64)[:, blk]                                   # [B, S]
    ok = (pos.reshape(1, -1) < lengths.reshape(B, 1).to(dev)) & (page >= 0) & ((pos // PAGE_SIZE) < MAX_BLOCKS).reshape(1, -1)
    page = page.clamp_min(0)
    off = (pos % PAGE_SIZE).reshape(1, -1).expand(B, -1)

    def gather(pages):
        out = pages[page, off]                                                   # [B, S, Hkv, D]
        return torch.where(ok.reshape(B, max_seq_len, 1, 1), out, torch.zeros((), dtype=pages.dtype, device=dev))

    return gather(K_pages), gather(V_pages)


# ---------------------------------------------------------------------------------------------
# decode attention
# ---------------------------------------------------------------------------------------------
def _validate_paged_quantized_decode_inputs(q, paged_qkv: PagedQuantizedKVCache):
    if q.ndim != 4:
        raise ValueError(f"q must be 4-D [B,1,Hq,D], got {tuple(q.shape)}")
    if q.shape[1] != 1:
        raise ValueError(f"q must have shape [B,1,Hq,D], got {tuple(q.shape)}")
    B, _, Hq, D = q.shape
    orig = paged_qkv.original_page_shape
    if orig is None:
        raise ValueError("original_page_shape is required for decode attention")
    NUM_PAGES, PAGE_SIZE, Hkv, D_cache = orig
    cache_B = paged_qkv.block_table.shape[0]
    if B != cache_B:
        raise ValueError(f"batch mismatch: q batch={B}, cache batch={cache_B}")
    if D != D_cache:
        raise ValueError(f"head_dim mismatch: q D={D}, cache D={D_cache}")
    validate_gqa_heads(Hq, Hkv)
    MAX_BLOCKS = paged_qkv.block_table.shape[1]
    return B, MAX_BLOCKS * PAGE_SIZE, PAGE_SIZE, MAX_BLOCKS, Hq, Hkv, D, NUM_PAGES


_workspaces: dict = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    """Scratch for the split-KV partial results, cached per device and stream (stream-ordered reuse)."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def paged_attention_launch(q3d, paged_qkv, scale, out=None, workspace=None, *, sink_tokens: int = 0, window_size: int = 0,
                           block_mask=None, block_size: int = 0):
    """q3d [B,Hq,D] -> [B,Hq,D]; all tensors already on one CUDA device.  ``window_size > 0`` restricts the
    attention to positions ``< sink_tokens`` or ``>= length - window_size``; ``block_mask`` (uint8 [q_blocks, k_blocks]
    on the device) with ``block_size`` to the keys j with ``block_mask[(length-1)//block_size, j//block_size]``."""
    B, Hq, D = q3d.shape
    NUM_PAGES, PAGE_SIZE, Hkv, _ = paged_qkv.original_page_shape
    MAX_BLOCKS = paged_qkv.block_table.shape[1]
    lib = _cabi.load()
    q3d = _cabi.contiguous(q3d)
    kq, vq = _cabi.contiguous(paged_qkv.k_pages_q), _cabi.contiguous(paged_qkv.v_pages_q)
    ks, vs = paged_qkv.k_scales, paged_qkv.v_scales
    if ks.dtype != vs.dtype or ks.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        ks, vs = ks.to(torch.float32), vs.to(torch.float32)
    ks, vs = _cabi.contiguous(ks), _cabi.contiguous(vs)
    bt = _cabi.contiguous(paged_qkv.block_table.to(torch.int32))
    ln = _cabi.contiguous(paged_qkv.lengths.reshape(B).to(torch.int32))
    if out is None:
        out = torch.empty_like(q3d)
    nbytes = lib.b200q_paged_gqa_workspace_bytes(B, Hq, Hkv, D)
    if workspace is None:
        workspace = _workspace(q3d.device, nbytes)
    args = (paged_qkv.bits, q3d.data_ptr(), kq.data_ptr(), vq.data_ptr(), ks.data_ptr(), vs.data_ptr(), bt.data_ptr(),
            ln.data_ptr(), out.data_ptr(), workspace.data_ptr(), workspace.numel(), B, Hq, Hkv, D, PAGE_SIZE, NUM_PAGES,
            MAX_BLOCKS, paged_qkv.group_size, float(scale), _cabi.dtype_code(q3d.dtype), _cabi.dtype_code(ks.dtype))
    if block_mask is not None:
        scratch = torch.empty(B * (MAX_BLOCKS + 1), dtype=torch.int32, device=q3d.device)
        _cabi.check(lib.b200q_paged_gqa_decode_block_sparse(
            *args[:11], block_mask.data_ptr(), block_mask.shape[0], block_mask.shape[1], int(block_size),
            scratch.data_ptr(), *args[11:], _cabi.stream()), "b200q_paged_gqa_decode_block_sparse")
    elif window_size > 0:
        _cabi.check(lib.b200q_paged_gqa_decode_window(*args, int(sink_tokens), int(window_size), _cabi.stream()),
                    "b200q_paged_gqa_decode_window")
    else:
        _cabi.check(lib.b200q_paged_gqa_decode(*args, _cabi.stream()), "b200q_paged_gqa_decode")
    return out


def reference_paged_quantized_kv_gqa_decode_attention(q, paged_qkv, *, scale: float | None = None):
    _cabi.reference_unavailable("reference_paged_quantized_kv_gqa_decode_attention")


def reference_sparse_paged_quantized_kv_gqa_decode_attention(q, paged_qkv, pattern, *, scale: float | None = None):
    _cabi.reference_unavailable("reference_sparse_paged_quantized_kv_gqa_decode_attention")


def paged_quantized_kv_gqa_decode_attention(q, paged_qkv: PagedQuantizedKVCache, *, scale: float | None = None,
                                            backend: str = "reference"):
    """q [B,1,Hq,D] -> [B,1,Hq,D].  Backends: ``"cuda"`` (picks the kernel from ``paged_qkv.bits``),
    or the reference's ``"metal_q8"`` / ``"metal_q4"`` with their bits precondition; the default
    ``"reference"`` names the pure-MLX path and raises here
    (ops/paged_quantized_kv_ops.py:632-661)."""
    B, MAX_S, PAGE_SIZE, MAX_BLOCKS, Hq, Hkv, D, NUM_PAGES = _validate_paged_quantized_decode_inputs(q, paged_qkv)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    name = backend.lower()
    if name == "reference":
        _cabi.reference_unavailable("paged_quantized_kv_gqa_decode_attention")
    if name == "metal_q8":
        if paged_qkv.bits != 8:
            raise ValueError(f"metal_q8 backend requires bits=8, got bits={paged_qkv.bits}")
    elif name == "metal_q4":
        if paged_qkv.bits != 4:
            raise ValueError(f"metal_q4 backend requires bits=4, got bits={paged_qkv.bits}")
    elif name not in ("cuda", "auto"):
        raise ValueError(f"backend must be one of 'reference', 'metal_q8', 'metal_q4', 'cuda', got {name!r}")
    if D > _MAX_HEAD_DIM:
        raise ValueError(f"{name} backend supports D <= {_MAX_HEAD_DIM}, got D={D}")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"q dtype must be float16 or bfloat16, got {q.dtype}")
    _cabi.require_cuda(q, paged_qkv.k_pages_q, paged_qkv.v_pages_q, paged_qkv.k_scales, paged_qkv.v_scales,
                       paged_qkv.block_table, paged_qkv.lengths)
    out = paged_attention_launch(q.reshape(B, Hq, D), paged_qkv, scale)
    return out.reshape(B, 1, Hq, D)


def sparse_paged_quantized_kv_gqa_decode_attention(q, paged_qkv: PagedQuantizedKVCache, pattern, *,
                                                   scale: float | None = None, backend: str = "cuda"):
    """Sparse decode over the paged quantized cache: q [B,1,Hq,D] -> [B,1,Hq,D].
    The reference has this as a pure-MLX scaffold only (reference_sparse_paged_quantized_kv_gqa_decode_attention,
    ops/paged_quantized_kv_ops.py:669-714); ``backend="reference"`` raises here like every reference path.
    ``pattern`` is a ``SparseAttentionPattern`` (dense, sliding_window, sliding_window_sink, block_sparse); every
    sequence needs at least one token, as in the reference.  A block_sparse row that hides every key yields zeros."""
    if not isinstance(pattern, SparseAttentionPattern):
        raise TypeError("pattern must be a SparseAttentionPattern")
    block_sparse = pattern.validate().pattern == "block_sparse"
    sink_tokens, window_size = (0, 0) if block_sparse else decode_window(pattern)
    B, MAX_S, PAGE_SIZE, MAX_BLOCKS, Hq, Hkv, D, NUM_PAGES = _validate_paged_quantized_decode_inputs(q, paged_qkv)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    name = backend.lower()
    if name == "reference":
        _cabi.reference_unavailable("sparse_paged_quantized_kv_gqa_decode_attention")
    if name not in ("cuda", "auto"):
        raise ValueError(f"backend must be one of 'reference', 'cuda', got {name!r}")
    if D > _MAX_HEAD_DIM:
        raise ValueError(f"{name} backend supports D <= {_MAX_HEAD_DIM}, got D={D}")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"q dtype must be float16 or bfloat16, got {q.dtype}")
    _cabi.require_cuda(q, paged_qkv.k_pages_q, paged_qkv.v_pages_q, paged_qkv.k_scales, paged_qkv.v_scales,
                       paged_qkv.block_table, paged_qkv.lengths)
    if block_sparse:
        mask, block_size = decode_block_mask(pattern, q.device)
        out = paged_attention_launch(q.reshape(B, Hq, D), paged_qkv, scale, block_mask=mask, block_size=block_size)
    else:
        out = paged_attention_launch(q.reshape(B, Hq, D), paged_qkv, scale, sink_tokens=sink_tokens, window_size=window_size)
    return out.reshape(B, 1, Hq, D)
