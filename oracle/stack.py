"""Oracle (test infrastructure): one decode step of a Llama-shaped q4/q8 stack with a paged
quantised KV cache, assembled from the reference's per-op reference functions.

The reference never wires its quantised paged cache into its layer stack
(ops/llama_stack_ops.py:129-130 raises for paged caches), so this composition follows
llama_layer_decode_step (ops/llama_layer_ops.py:234-428) for the order of operations and rounding
points - rms_norm -> QKV matvec -> split + interleaved RoPE (ops/gqa_ops.py:148-160,
ops/rope_ops.py:61-75) -> attention -> O matvec -> residual add -> quantized_mlp_block with a zero
residual - and swaps its fp16 cache for: append the new K/V row quantised like
_quantize_group_symmetric_8/_4 (ops/paged_quantized_kv_ops.py:146-175), then the paged quantised
GQA decode attention over positions [0, pos].
"""
from __future__ import annotations

import torch

from .elementwise_ops import reference_residual_add, reference_rms_norm
from .mlp_block_ops import reference_quantized_linear, reference_quantized_mlp_block
from .paged_quantized_kv_ops import (OraclePagedKV, _quantize_groups_symmetric,
                                     reference_paged_quantized_kv_gqa_decode_attention)
from .quant_ops import pack_q4


def rope_tables(head_dim: int, theta: float, length: int):
    """cos/sin [length, head_dim/2] fp32 (models/llama_config.py:107-124)."""
    inv_freq = 1.0 / (float(theta) ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / float(head_dim)))
    freqs = torch.arange(length, dtype=torch.float32).reshape(length, 1) * inv_freq.reshape(1, head_dim // 2)
    return torch.cos(freqs), torch.sin(freqs)


def apply_rope_rows(x, cos, sin, positions):
    """x [B, H, D] at per-sequence positions; pairs (2i, 2i+1) (ops/rope_ops.py:61-75)."""
    c = cos[positions.long()].to(torch.float32).unsqueeze(1)      # [B, 1, D/2]
    s = sin[positions.long()].to(torch.float32).unsqueeze(1)
    xe = x[..., 0::2].to(torch.float32)
    xo = x[..., 1::2].to(torch.float32)
    ye = xe * c - xo * s
    yo = xe * s + xo * c
    return torch.stack([ye, yo], dim=-1).reshape(x.shape).to(x.dtype)


def append_kv(cache: OraclePagedKV, k_rows, v_rows, positions):
    """Quantise k_rows / v_rows [B, Hkv, D] and store them at position positions[b] of sequence b."""
    _, P, Hkv, D = cache.original_page_shape
    limit, offset = (127, 128) if cache.bits == 8 else (7, 8)
    for rows, codes_dst, scales_dst in ((k_rows, cache.k_pages_q, cache.k_scales), (v_rows, cache.v_pages_q, cache.v_scales)):
        codes, scales = _quantize_groups_symmetric(rows.to(torch.float32), cache.group_size, limit, offset)
        if cache.bits == 4:
            codes = pack_q4(codes.reshape(-1, D)).reshape(rows.shape[0], Hkv, (D + 1) // 2)
        for b in range(rows.shape[0]):
            pos = int(positions[b])
            page = int(cache.block_table[b, pos // P])
            if page < 0:
                continue
            codes_dst[page, pos % P] = codes[b]
            scales_dst[page, pos % P] = scales[b]


def layer_decode_step(h, w, cache, cos, sin, positions, cfg):
    """h [B, 1, hidden] -> [B, 1, hidden]; mutates ``cache`` (append) but not its lengths."""
    B = h.shape[0]
    Hq, Hkv, D = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    bits, G, eps = cfg["bits"], cfg["group_size"], cfg["eps"]
    x_norm = reference_rms_norm(h, w["input_norm"], eps=eps)
    qkv = reference_quantized_linear(x_norm, *w["qkv"], bits=bits, group_size=G).reshape(B, Hq + 2 * Hkv, D)
    q = apply_rope_rows(qkv[:, :Hq], cos, sin, positions)
    k = apply_rope_rows(qkv[:, Hq:Hq + Hkv], cos, sin, positions)
    v = qkv[:, Hq + Hkv:]
    append_kv(cache, k, v, positions)
    saved = cache.lengths
    cache.lengths = (positions + 1).to(torch.int32)
    attn = reference_paged_quantized_kv_gqa_decode_attention(q.reshape(B, 1, Hq, D), cache)
    cache.lengths = saved
    attn_proj = reference_quantized_linear(attn.reshape(B, 1, Hq * D), *w["o"], bits=bits, group_size=G)
    h2 = reference_residual_add(h, attn_proj)
    gw, gs, gz = w["gate"]
    uw, us, uz = w["up"]
    dw, ds, dz = w["down"]
    return reference_quantized_mlp_block(h2, torch.zeros_like(h2), w["post_norm"], gw, gs, uw, us, dw, ds,
                                         gate_zeros=gz, up_zeros=uz, down_zeros=dz, bits=bits, group_size=G, eps=eps)


def stack_decode_step(token_ids, embedding, layers, caches, final_norm, cos, sin, positions, cfg):
    """token_ids [B] -> final-normed hidden [B, 1, hidden] (logits are not part of the benchmark)."""
    h = embedding[token_ids.long()].unsqueeze(1)
    for w, cache in zip(layers, caches):
        h = layer_decode_step(h, w, cache, cos, sin, positions, cfg)
    return reference_rms_norm(h, final_norm, eps=cfg["eps"])
