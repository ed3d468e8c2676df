"""Seeded synthetic inputs with the shapes and value distributions of the decode benchmarks.

The reference publishes no dataset and no checkpoint for this path; every benchmark
configuration is defined by a distribution (activations N(0,1), weights N(0,0.02),
K/V N(0,1)) and a quantisation rule.  These generators produce exactly those tensors from a
``torch.Generator`` seed, on any device.
"""
from __future__ import annotations

import math

import torch


def _randn(shape, seed, device, std=1.0):
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    # CPU generation keeps the stream identical whatever device the tensors end up on.
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(device)


def activations(shape, seed, device="cpu", dtype=torch.float16):
    return _randn(shape, seed, device).to(dtype)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] codes in 0..15 -> [..., ceil(K/2)] bytes, low nibble = even k
    (layout of pack_q4, reference ops/quant_ops.py:166-176)."""
    if codes.shape[-1] % 2:
        codes = torch.nn.functional.pad(codes, (0, 1))
    c = codes.to(torch.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).contiguous()


def quantize_affine(weight: torch.Tensor, bits: int, group_size: int, scale_dtype=torch.float16):
    """Group-wise affine quantisation along the last axis.

    scale = (max - min) / (2^bits - 1), code = clip(rint((w - min) / scale), 0, 2^bits - 1).
    Returned in the reference's dequant convention ``(code - zero) * scale``
    (ops/quant_ops.py:205-212): ``zeros = -min / scale``.  Codes are uint8; 4-bit codes are
    packed two per byte.
    """
    if bits not in (4, 8):
        raise ValueError(f"bits must be 4 or 8, got {bits}")
    N, K = weight.shape
    groups = math.ceil(K / group_size)
    pad = groups * group_size - K
    w = weight.to(torch.float32)
    if pad:
        w = torch.cat([w, w[:, -1:].expand(N, pad)], dim=1)
    wg = w.reshape(N, groups, group_size)
    lo = wg.amin(dim=-1, keepdim=True)
    hi = wg.amax(dim=-1, keepdim=True)
    qmax = float(2 ** bits - 1)
    scale = ((hi - lo) / qmax).clamp_min(1e-8)
    codes = torch.round((wg - lo) / scale).clamp(0, qmax).to(torch.uint8).reshape(N, groups * group_size)[:, :K]
    zeros = (-lo / scale).squeeze(-1)
    scales = scale.squeeze(-1)
    packed = pack_nibbles(codes) if bits == 4 else codes.contiguous()
    return packed, scales.to(scale_dtype).contiguous(), zeros.to(scale_dtype).contiguous()


def quantized_weight(N, K, bits, group_size, seed, device="cpu", std=0.02, scale_dtype=torch.float16):
    """W ~ N(0, std) [N out, K in] quantised with :func:`quantize_affine`."""
    w = _randn((N, K), seed, device, std=std)
    return quantize_affine(w, bits, group_size, scale_dtype)


def quantize_kv_symmetric(pages: torch.Tensor, bits: int, group_size: int):
    """Symmetric scale-only KV quantisation per (page, slot, head, group along D), fp16 scales:
    the rule of the reference cache (ops/paged_quantized_kv_ops.py:146-153, 168-175).
    Returns (codes [.., D or ceil(D/2)], scales [.., ceil(D/G)])."""
    limit, offset = (127, 128) if bits == 8 else (7, 8)
    D = pages.shape[-1]
    groups = (D + group_size - 1) // group_size
    pad = groups * group_size - D
    v = pages.to(torch.float32)
    if pad:
        v = torch.nn.functional.pad(v, (0, pad))
    v = v.reshape(*pages.shape[:-1], groups, group_size)
    scale = v.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8) / float(limit)
    codes = (torch.round(v / scale).clamp(-limit, limit) + offset).to(torch.uint8)
    codes = codes.reshape(*pages.shape[:-1], groups * group_size)[..., :D]
    if bits == 4:
        codes = pack_nibbles(codes)
    return codes.contiguous(), scale.squeeze(-1).to(torch.float16).contiguous()


def paged_kv_case(B, Hkv, D, page_size, num_pages, min_len, max_len, bits, group_size, seed, device="cpu"):
    """Random K/V pages ~N(0,1), lengths uniform in [min_len, max_len], block tables drawn from one
    random permutation of the page pool dealt out contiguously to the sequences; unused
    block-table entries are -1."""
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    lengths = torch.randint(min_len, max_len + 1, (B,), generator=g, dtype=torch.int32)
    blocks = (lengths + page_size - 1) // page_size
    max_blocks = max(1, (max_len + page_size - 1) // page_size)
    if int(blocks.sum()) > num_pages:
        raise ValueError("page pool too small for the sampled lengths")
    perm = torch.randperm(num_pages, generator=g).to(torch.int32)
    block_table = torch.full((B, max_blocks), -1, dtype=torch.int32)
    cursor = 0
    for b in range(B):
        n = int(blocks[b])
        block_table[b, :n] = perm[cursor:cursor + n]
        cursor += n
    shape = (num_pages, page_size, Hkv, D)
    k_codes, k_scales = quantize_kv_symmetric(_randn(shape, seed + 1, device), bits, group_size)
    v_codes, v_scales = quantize_kv_symmetric(_randn(shape, seed + 2, device), bits, group_size)
    return {
        "k_pages_q": k_codes, "v_pages_q": v_codes, "k_scales": k_scales, "v_scales": v_scales,
        "block_table": block_table.to(device), "lengths": lengths.to(device),
        "bits": bits, "page_size": page_size, "group_size": group_size, "original_page_shape": shape,
    }
