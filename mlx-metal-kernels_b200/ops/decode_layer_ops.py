"""Decode-layer glue around the hot-path operators: fused RMSNorm + quantized projection, and
QKV split + RoPE + quantised KV append.  These are the pieces of the reference's
llama_layer_decode_step (ops/llama_layer_ops.py:234-428) that sit between the matvec and the
attention kernels."""
from __future__ import annotations

import torch

from . import _cabi


def norm_quantized_linear(x, norm_weight, w, scales, zeros=None, *, residual_in=None, bits=4, group_size=32, eps=1e-5,
                          return_normed=False):
    """y = W rmsnorm(x + residual_in) for rows x [R, K] (fp16/bf16); one launch on the tensor-core path."""
    _cabi.require_cuda(x, norm_weight, w, scales, zeros, residual_in)
    x = _cabi.contiguous(x)
    w = _cabi.contiguous(w.to(torch.uint8))
    scales, zeros = _cabi.scale_pair(scales, zeros)
    norm_weight = _cabi.contiguous(norm_weight)
    residual_in = None if residual_in is None else _cabi.contiguous(residual_in.to(x.dtype))
    R, K = x.shape
    N = w.shape[0]
    y = torch.empty((R, N), dtype=x.dtype, device=x.device)
    normed = torch.empty_like(x)           # also the staging buffer of the generic (odd-shape) route
    _cabi.check(
        _cabi.load().b200q_norm_qmatvec(bits, x.data_ptr(), _cabi.ptr(residual_in), norm_weight.data_ptr(),
                                        _cabi.dtype_code(norm_weight.dtype), float(eps), None, normed.data_ptr(),
                                        w.data_ptr(), scales.data_ptr(), _cabi.ptr(zeros), None, y.data_ptr(), R, N, K,
                                        group_size, _cabi.dtype_code(x.dtype), _cabi.dtype_code(scales.dtype),
                                        _cabi.stream()),
        "b200q_norm_qmatvec",
    )
    return (y, normed) if return_normed else y


def rope_kv_append(qkv, cos, sin, positions, paged_qkv, n_heads: int):
    """qkv [B, (Hq + 2 Hkv) * D] fp16 -> q_rot [B, Hq, D]; appends the rotated k and the v row of every
    sequence to ``paged_qkv`` (a PagedQuantizedKVCache, modified in place) at ``positions[b]``."""
    NUM_PAGES, P, Hkv, D = paged_qkv.original_page_shape
    B = qkv.shape[0]
    _cabi.require_cuda(qkv, cos, sin, positions, paged_qkv.k_pages_q, paged_qkv.block_table)
    if qkv.dtype != torch.float16 or paged_qkv.k_scales.dtype != torch.float16:
        raise TypeError("rope_kv_append needs fp16 activations and fp16 cache scales")
    qkv = _cabi.contiguous(qkv)
    cos = _cabi.contiguous(cos.to(torch.float32))
    sin = _cabi.contiguous(sin.to(torch.float32))
    positions = _cabi.contiguous(positions.to(torch.int32))
    bt = paged_qkv.block_table
    if bt.dtype != torch.int32 or not bt.is_contiguous():
        raise TypeError("block_table must be a contiguous int32 tensor")
    q_out = torch.empty((B, n_heads, D), dtype=torch.float16, device=qkv.device)
    _cabi.check(
        _cabi.load().b200q_rope_kv_append(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), positions.data_ptr(),
                                          bt.data_ptr(), q_out.data_ptr(), paged_qkv.k_pages_q.data_ptr(),
                                          paged_qkv.v_pages_q.data_ptr(), paged_qkv.k_scales.data_ptr(),
                                          paged_qkv.v_scales.data_ptr(), paged_qkv.bits, B, n_heads, Hkv, D, P, NUM_PAGES,
                                          bt.shape[1], paged_qkv.group_size, cos.shape[0], _cabi.stream()),
        "b200q_rope_kv_append",
    )
    return q_out


def rope_append_attention(qkv, cos, sin, positions, paged_qkv, n_heads: int, *, scale: float | None = None):
    """The attention stage of a decode layer in one call: split the fused qkv rows [B, (Hq + 2 Hkv) * D], rotate q and
    k at ``positions[b]``, append the quantised k / v of the new token to ``paged_qkv`` (modified in place; its
    ``lengths`` must already count the new token) and attend over the cache.  Returns [B, Hq, D].  Small batches run
    as a single kernel (one thread-block cluster per sequence and kv head); others as append + split-KV attention."""
    import math
    NUM_PAGES, P, Hkv, D = paged_qkv.original_page_shape
    B = qkv.shape[0]
    _cabi.require_cuda(qkv, cos, sin, positions, paged_qkv.k_pages_q, paged_qkv.block_table, paged_qkv.lengths)
    if qkv.dtype != torch.float16 or paged_qkv.k_scales.dtype != torch.float16:
        raise TypeError("rope_append_attention needs fp16 activations and fp16 cache scales")
    qkv = _cabi.contiguous(qkv)
    cos = _cabi.contiguous(cos.to(torch.float32))
    sin = _cabi.contiguous(sin.to(torch.float32))
    positions = _cabi.contiguous(positions.to(torch.int32))
    bt = paged_qkv.block_table
    ln = paged_qkv.lengths
    if bt.dtype != torch.int32 or not bt.is_contiguous() or ln.dtype != torch.int32:
        raise TypeError("block_table and lengths must be contiguous int32 tensors")
    lib = _cabi.load()
    out = torch.empty((B, n_heads, D), dtype=torch.float16, device=qkv.device)
    q_scratch = torch.empty_like(out)
    ws = torch.empty(max(16, lib.b200q_paged_gqa_workspace_bytes(B, n_heads, Hkv, D)), dtype=torch.uint8, device=qkv.device)
    _cabi.check(
        lib.b200q_rope_append_paged_gqa_decode(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), positions.data_ptr(),
                                               cos.shape[0], paged_qkv.bits, paged_qkv.k_pages_q.data_ptr(),
                                               paged_qkv.v_pages_q.data_ptr(), paged_qkv.k_scales.data_ptr(),
                                               paged_qkv.v_scales.data_ptr(), bt.data_ptr(), ln.reshape(B).data_ptr(),
                                               out.data_ptr(), q_scratch.data_ptr(), ws.data_ptr(), ws.numel(), B, n_heads,
                                               Hkv, D, P, NUM_PAGES, bt.shape[1], paged_qkv.group_size,
                                               float(scale if scale is not None else 1.0 / math.sqrt(D)), _cabi.stream()),
        "b200q_rope_append_paged_gqa_decode",
    )
    return out
