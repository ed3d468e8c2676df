"""GPU parity: contiguous q4/q8 KV cache (quantise, dequantise, GQA decode attention) against the CPU
oracle.  Bounds: codes, scales and dequantised values bit-exact; attention max |out - oracle| <= 2e-3
in fp16 (K/V ~ N(0,1))."""
import numpy as np
import pytest
import torch

from helpers import qkv_ops
from oracle import quantized_kv_cache_ops as oc

pytestmark = pytest.mark.gpu
ATOL = 2e-3


def _randn(shape, seed, dtype=torch.float16):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(dtype)


def _to_device(cache, device):
    return qkv_ops.QuantizedKVCache(k_q=cache.k_q.to(device), v_q=cache.v_q.to(device),
                                    k_scales=cache.k_scales.to(device), v_scales=cache.v_scales.to(device),
                                    bits=cache.bits, group_size=cache.group_size, original_shape=cache.original_shape)


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("B,MAX_S,Hq,Hkv,D,lengths", [
    (1, 16, 4, 2, 16, None), (2, 16, 4, 1, 64, None), (1, 16, 4, 4, 128, None),   # tests/test_quantized_kv_decode_attention_metal.py shapes
    (3, 64, 8, 2, 128, [64, 17, 1]),          # multiple of 16: pages of 16 tokens, tensor-core kernel
    (2, 256, 32, 8, 128, [256, 100]),
    (2, 50, 8, 2, 128, [50, 33]),             # not a multiple of 16: one page per sequence
    (2, 37, 6, 3, 48, 20),                    # scalar length, short last group
])
def test_attention_matches_oracle(cuda, bits, B, MAX_S, Hq, Hkv, D, lengths):
    K, V = _randn((B, MAX_S, Hkv, D), 11), _randn((B, MAX_S, Hkv, D), 12)
    cache = oc.quantize_kv_cache(K, V, bits=bits, group_size=32)
    q = _randn((B, 1, Hq, D), 13)
    want = oc.reference_quantized_kv_gqa_decode_attention(q, cache, lengths)
    for backend in ("cuda", f"metal_q{bits}"):
        got = qkv_ops.quantized_kv_gqa_decode_attention(q.to(cuda), _to_device(cache, cuda), lengths, backend=backend)
        assert got.shape == q.shape and got.dtype == q.dtype
        err = float((got.cpu().float() - want.float()).abs().max())
        assert err <= ATOL, err


@pytest.mark.parametrize("bits", [8, 4])
def test_attention_bf16_queries_and_device_lengths(cuda, bits):
    B, MAX_S, Hq, Hkv, D = 2, 48, 8, 4, 64
    K, V = _randn((B, MAX_S, Hkv, D), 21), _randn((B, MAX_S, Hkv, D), 22)
    cache = oc.quantize_kv_cache(K, V, bits=bits, group_size=32)
    q = _randn((B, 1, Hq, D), 23, torch.bfloat16)
    lengths = torch.tensor([48, 5], dtype=torch.int32)
    want = oc.reference_quantized_kv_gqa_decode_attention(q, cache, lengths)
    got = qkv_ops.quantized_kv_gqa_decode_attention(q.to(cuda), _to_device(cache, cuda), lengths.to(cuda), backend="cuda")
    # bf16 output: half an ulp of the largest output on top of the fp16 bound
    bound = ATOL + float(want.float().abs().max()) * 2.0 ** -8
    assert float((got.cpu().float() - want.float()).abs().max()) <= bound


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("tag", ["gqa", "mqa", "d16"])
def test_attention_matches_metal_kernel_fixture(cuda, golden, bits, tag):
    key = f"mtl_cattn_q{bits}_{tag}"
    g = {n: torch.from_numpy(np.ascontiguousarray(golden[f"{key}_{n}"]))
         for n in ("q", "kq", "vq", "ks", "vs", "lengths", "out")}
    shape = tuple(int(v) for v in golden[f"{key}_shape"])
    cache = qkv_ops.QuantizedKVCache(k_q=g["kq"].to(cuda), v_q=g["vq"].to(cuda), k_scales=g["ks"].to(cuda),
                                     v_scales=g["vs"].to(cuda), bits=bits, group_size=32, original_shape=shape)
    got = qkv_ops.quantized_kv_gqa_decode_attention(g["q"].to(cuda), cache, g["lengths"].to(cuda), backend="cuda")
    want = g["out"].float()
    assert bool(((got.cpu().float() - want).abs() <= 2e-3 + want.abs() * 2.0 ** -10).all())


@pytest.mark.parametrize("bits", [8, 4])
def test_quantise_and_dequantise_are_bit_exact(cuda, bits):
    B, MAX_S, Hkv, D = 2, 19, 3, 80
    K, V = _randn((B, MAX_S, Hkv, D), 31), _randn((B, MAX_S, Hkv, D), 32)
    lengths = [19, 6]
    want = oc.quantize_kv_cache(K, V, bits=bits, group_size=32, lengths=lengths)
    got = qkv_ops.quantize_kv_cache(K.to(cuda), V.to(cuda), qkv_ops.QuantizedKVCacheConfig(bits=bits, group_size=32),
                                    lengths=lengths)
    for name in ("k_q", "v_q", "k_scales", "v_scales"):
        assert torch.equal(getattr(got, name).cpu(), getattr(want, name)), name
    assert got.original_shape == (B, MAX_S, Hkv, D) and got.bits == bits
    Kd, Vd = qkv_ops.dequantize_kv_cache(got)
    Kw, Vw = oc.dequantize_kv_cache(want)
    assert torch.equal(Kd.cpu(), Kw) and torch.equal(Vd.cpu(), Vw)
    report = qkv_ops.quantized_kv_error(K.to(cuda)[:1], V.to(cuda)[:1], qkv_ops.QuantizedKVCache(
        k_q=got.k_q[:1], v_q=got.v_q[:1], k_scales=got.k_scales[:1], v_scales=got.v_scales[:1], bits=bits,
        group_size=32, original_shape=(1, MAX_S, Hkv, D)))
    assert 0.0 < report["k_rmse"] < (0.02 if bits == 8 else 0.3) and report["compression_ratio"] > 1.0


def test_zero_length_sequence_gives_zeros(cuda):
    B, MAX_S, Hq, Hkv, D = 2, 32, 4, 2, 128
    cache = oc.quantize_kv_cache(_randn((B, MAX_S, Hkv, D), 41), _randn((B, MAX_S, Hkv, D), 42), bits=8, group_size=32)
    q = _randn((B, 1, Hq, D), 43)
    got = qkv_ops.quantized_kv_gqa_decode_attention(q.to(cuda), _to_device(cache, cuda), [0, 32], backend="cuda")
    assert float(got[0].abs().max()) == 0.0
    want = oc.reference_quantized_kv_gqa_decode_attention(q, cache, [0, 32])
    assert float((got[1].cpu().float() - want[1].float()).abs().max()) <= ATOL


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("MAX_S,lengths,sink,window", [(128, [128, 45], 4, 32), (128, [77, 128], 0, 16), (50, [50, 9], 2, 8)])
def test_sliding_window_decode_matches_oracle(cuda, bits, MAX_S, lengths, sink, window):
    from helpers import sparse_ops
    B, Hq, Hkv, D = 2, 8, 2, 128
    cache = oc.quantize_kv_cache(_randn((B, MAX_S, Hkv, D), 51), _randn((B, MAX_S, Hkv, D), 52), bits=bits, group_size=32)
    q = _randn((B, 1, Hq, D), 53)
    want = oc.reference_quantized_kv_gqa_decode_attention(q, cache, lengths, window=(sink, window))
    pattern = sparse_ops.SparseAttentionPattern("sliding_window_sink" if sink else "sliding_window", window_size=window,
                                                sink_tokens=sink)
    got = qkv_ops.quantized_kv_sparse_gqa_decode_attention(q.to(cuda), _to_device(cache, cuda), lengths, pattern,
                                                           backend="cuda")
    assert float((got.cpu().float() - want.float()).abs().max()) <= ATOL
