"""CPU-side checks: the C ABI surface, argument validation, backend-flag handling and the data
helpers.  No kernel is launched here."""
import dataclasses
import re

import pytest
import torch

from helpers import (act_ops, cabi, fused_ops, mlp_ops, norm_ops, pkv_ops, pq_ops, qkv_ops, quant_ops, random_quant_case,
                     sparse_ops, synth)
from oracle import paged_quantized_kv_ops as opq, quant_ops as oq, quantized_kv_cache_ops as ocq
from oracle import sparse_attention_ops as osparse


def test_library_exports_every_declared_symbol():
    declared = cabi.header_functions()
    assert declared == sorted(cabi.SIGNATURES), "include/b200q.h and the ctypes table disagree"
    lib = cabi.load()
    for name in declared:
        assert hasattr(lib, name)
    assert lib.b200q_version() >= 100
    assert b"workspace" in lib.b200q_strerror(-4)


def test_header_cites_reference_sites():
    text = cabi.HEADER_PATH.read_text()
    for needle in ("ops/quant_ops.py", "ops/mlp_block_ops.py", "ops/paged_quantized_kv_ops.py", "ops/paged_kv_ops.py"):
        assert needle in text
    assert re.search(r"ops/quant_ops\.py:\d+", text)


def test_pack_unpack_roundtrip_and_layout():
    codes = torch.randint(0, 16, (4, 64), dtype=torch.int32).to(torch.uint8)
    packed = quant_ops.pack_q4(codes)
    assert packed.shape == (4, 32) and packed.dtype == torch.uint8
    assert torch.equal(packed, oq.pack_q4(codes))
    assert torch.equal(quant_ops.unpack_q4_reference(packed, K=64), codes)
    odd = torch.randint(0, 16, (3, 7), dtype=torch.int32).to(torch.uint8)
    assert quant_ops.pack_q4(odd).shape == (3, 4)
    assert torch.equal(quant_ops.unpack_q4_reference(quant_ops.pack_q4(odd), K=7), odd)
    with pytest.raises(ValueError):
        quant_ops.pack_q4(torch.zeros(4, dtype=torch.uint8))


@pytest.mark.parametrize("bits", [4, 8])
def test_matvec_validation_errors(bits):
    codes, scales, zeros = random_quant_case(bits, 32, 64, 32, 1)
    x = torch.randn(2, 64).to(torch.float16)
    fn = quant_ops.q4_matvec_decode if bits == 4 else quant_ops.q8_matvec_decode
    with pytest.raises(TypeError, match="x dtype must be float16 or bfloat16"):
        fn(x.float(), codes, scales, zeros)
    with pytest.raises(ValueError, match=r"x must have shape \[B,K\] or \[B,1,K\]"):
        fn(x.reshape(1, 2, 64), codes, scales, zeros)
    with pytest.raises(ValueError, match="scales must have shape"):
        fn(x, codes, scales[:, :1], zeros, group_size=32)
    with pytest.raises(ValueError, match="zeros must have shape"):
        fn(x, codes, scales, zeros[:1], group_size=32)
    with pytest.raises(ValueError, match="group_size must be positive"):
        fn(x, codes, scales, zeros, group_size=0)
    with pytest.raises(ValueError, match="backend must be one of"):
        fn(x, codes, scales, zeros, backend="vulkan")
    bad_k = torch.randn(2, 66).to(torch.float16)
    with pytest.raises(ValueError):
        fn(bad_k, codes, scales, zeros)


def test_reference_backend_and_safe_mode_are_refused(monkeypatch):
    codes, scales, zeros = random_quant_case(4, 32, 64, 32, 2)
    x = torch.randn(1, 64).to(torch.float16)
    with pytest.raises(cabi.ReferenceBackendUnavailable):
        quant_ops.q4_matvec_decode(x, codes, scales, zeros, backend="reference")
    with pytest.raises(cabi.ReferenceBackendUnavailable):
        quant_ops.dequant_q4(codes, scales, zeros, backend="reference")
    with pytest.raises(cabi.ReferenceBackendUnavailable):
        quant_ops.reference_q4_matvec_decode(x, codes, scales, zeros)
    monkeypatch.setenv("MLX_METAL_CI_SAFE_MODE", "1")
    with pytest.raises(cabi.ReferenceBackendUnavailable):
        quant_ops.q4_matvec_decode(x, codes, scales, zeros, backend="metal_tiled")
    # dequant in safe mode is refused before the backend name is even looked at (reference order)
    with pytest.raises(cabi.ReferenceBackendUnavailable):
        quant_ops.dequant_q4(codes, scales, zeros, backend="bogus")


def test_cuda_backend_never_falls_back_to_cpu():
    codes, scales, zeros = random_quant_case(4, 32, 64, 32, 3)
    x = torch.randn(1, 64).to(torch.float16)
    for backend in ("auto", "cuda", "metal", "metal_parallel", "metal_tiled"):
        with pytest.raises(cabi.B200QError, match="no CPU route"):
            quant_ops.q4_matvec_decode(x, codes, scales, zeros, backend=backend)
    with pytest.raises(cabi.B200QError, match="no CPU route"):
        quant_ops.dequant_q4(codes, scales, zeros)


def test_dequant_validation_errors():
    codes, scales, zeros = random_quant_case(4, 4, 64, 32, 4)
    with pytest.raises(TypeError, match="out_dtype must be float16 or bfloat16"):
        quant_ops.dequant_q4(codes, scales, zeros, out_dtype=torch.float32)
    with pytest.raises(ValueError, match="packed must be 2-D"):
        quant_ops.dequant_q4(codes[0], scales, zeros)
    with pytest.raises(ValueError, match="backend must be one of"):
        quant_ops.dequant_q8(torch.zeros(4, 64, dtype=torch.uint8), scales, zeros, backend="nope")
    with pytest.raises(ValueError, match="bits must be 4 or 8"):
        quant_ops.groupwise_dequant(codes, scales, zeros, bits=3)


def test_gate_up_and_linear_validation_errors():
    gw, gs, _ = random_quant_case(4, 128, 64, 32, 5, zeros=None)
    uw, us, _ = random_quant_case(4, 128, 64, 32, 6, zeros=None)
    x = torch.randn(1, 1, 64).to(torch.float16)
    with pytest.raises(ValueError, match="backend must be one of"):
        mlp_ops.quantized_gate_up_projection(x, gw, gs, uw, us, backend="opencl")
    with pytest.raises(ValueError, match="bits must be 4 or 8"):
        mlp_ops.quantized_gate_up_projection(x, gw, gs, uw, us, bits=3)
    with pytest.raises(ValueError, match="bits must be 4 or 8"):
        mlp_ops.quantized_linear(x, gw, gs, bits=3)
    with pytest.raises(ValueError, match="scales must have shape"):
        mlp_ops.quantized_linear(x, gw, gs[:, :1], bits=4, group_size=32)
    with pytest.raises(ValueError, match="identical shapes"):
        quant_ops.q4_gate_up_matvec_tiled(x, gw, uw[:64], gs, us[:64])
    with pytest.raises(cabi.ReferenceBackendUnavailable):
        mlp_ops.quantized_gate_up_projection(x, gw, gs, uw, us, backend="reference")


def test_mlp_block_validation_and_presets():
    assert mlp_ops._resolve_mlp_backends(backend_preset="fused_experimental") == (
        "metal", "metal_gate_up_tiled", "metal_fused", "metal")
    assert mlp_ops._resolve_mlp_backends(backend_preset="parallel")[1] == "metal_parallel"
    with pytest.raises(ValueError, match="backend_preset must be one of"):
        mlp_ops._resolve_mlp_backends(backend_preset="turbo")
    x = torch.randn(1, 1, 64).to(torch.float16)
    w = torch.ones(64)
    gw, gs, _ = random_quant_case(4, 128, 64, 32, 7, zeros=None)
    dw, ds, _ = random_quant_case(4, 64, 128, 32, 8, zeros=None)
    with pytest.raises(ValueError, match="identical shapes"):
        mlp_ops.quantized_mlp_block(x, x[:, :, :32], w, gw, gs, gw, gs, dw, ds)
    with pytest.raises(ValueError, match=r"shape \[B,S,D\]"):
        mlp_ops.quantized_mlp_block(x[0], x[0], w, gw, gs, gw, gs, dw, ds)
    with pytest.raises(ValueError, match="norm_weight must have shape"):
        mlp_ops.quantized_mlp_block(x, x, w[:32], gw, gs, gw, gs, dw, ds)
    with pytest.raises(cabi.ReferenceBackendUnavailable):
        mlp_ops.quantized_mlp_block(x, x, w, gw, gs, gw, gs, dw, ds, backend_preset="reference")
    with pytest.raises(ValueError, match="bits must be 4 or 8"):
        mlp_ops.quantized_mlp_block(x, x, w, gw, gs, gw, gs, dw, ds, bits=3, backend_preset="tiled")


def test_elementwise_validation():
    g = torch.randn(2, 3, 8).to(torch.float16)
    with pytest.raises(ValueError, match="identical shapes"):
        act_ops.swiglu(g, g[:, :2])
    with pytest.raises(TypeError):
        act_ops.swiglu(g.float(), g.float())
    with pytest.raises(ValueError, match="backend must be one of"):
        act_ops.fused_swiglu(g, g, backend="x")
    with pytest.raises(ValueError, match="requires"):
        act_ops.fused_swiglu(g[0], g[0], backend="metal")
    with pytest.raises(ValueError, match="weight shape must be"):
        norm_ops.rms_norm(g, torch.ones(4))
    with pytest.raises(ValueError, match="identical shapes"):
        fused_ops.residual_add(g, g[:1])
    with pytest.raises(TypeError):
        fused_ops.residual_add(g.float(), g.float())


def test_paged_config_and_cache_validation():
    C = pq_ops.PagedQuantizedKVConfig
    assert dataclasses.asdict(C()) == dict(bits=8, page_size=16, group_size=32, symmetric=True, with_zeros=False,
                                           scale_dtype="float16", layout="paged")
    with pytest.raises(ValueError):
        C(bits=3).validate()
    with pytest.raises(ValueError):
        C(page_size=0).validate()
    with pytest.raises(ValueError):
        C(group_size=0).validate()
    with pytest.raises(NotImplementedError):
        C(symmetric=False).validate()
    with pytest.raises(NotImplementedError):
        C(with_zeros=True).validate()
    with pytest.raises(ValueError):
        C(layout="flat").validate()


@pytest.mark.parametrize("bits,D,G", [(8, 32, 32), (4, 32, 32), (4, 17, 16), (8, 16, 32)])
def test_paged_cache_container_accounts_bytes(bits, D, G):
    """The container's shape / byte accounting on a cache quantised by the oracle; the quantiser itself is a CUDA
    kernel (compared with the oracle in the GPU tests) and refuses CPU tensors."""
    torch.manual_seed(bits * 100 + D)
    K = torch.randn(6, 4, 2, D).to(torch.float16)
    V = torch.randn(6, 4, 2, D).to(torch.float16)
    bt = torch.arange(6, dtype=torch.int32).reshape(2, 3)
    ln = torch.tensor([12, 9], dtype=torch.int32)
    with pytest.raises(cabi.B200QError, match="no CPU route"):
        pq_ops.quantize_kv_pages(K, V, bt, ln, pq_ops.PagedQuantizedKVConfig(bits=bits, page_size=4, group_size=G))
    ref = opq.quantize_kv_pages(K, V, bt, ln, bits=bits, page_size=4, group_size=G)
    cache = pq_ops.PagedQuantizedKVCache(**{f.name: getattr(ref, f.name) for f in dataclasses.fields(ref)})
    dp = (D + 1) // 2 if bits == 4 else D
    groups = (D + G - 1) // G
    assert cache.shapes()["k_pages_q"] == (6, 4, 2, dp) and cache.shapes()["k_scales"] == (6, 4, 2, groups)
    assert cache.k_scales.dtype == torch.float16 and cache.num_pages() == 6
    expected = 2 * 6 * 4 * 2 * dp + 2 * 6 * 4 * 2 * groups * 2 + bt.numel() * 4 + ln.numel() * 4
    assert cache.memory_bytes() == expected
    assert 1.0 < cache.compression_ratio() < 10.0
    cache.validate()
    # dequantised oracle values are within half a step (plus fp16 rounding) of the originals
    Kd, _ = opq.dequantize_kv_pages(ref)
    step = ref.k_scales.float().repeat_interleave(G, dim=-1)[..., :D]
    assert bool(((Kd.float() - K.float()).abs() <= 0.5 * step * 1.01 + 2e-3).all())


def test_contiguous_pages_roundtrip():
    torch.manual_seed(0)
    K = torch.randn(2, 8, 2, 16).to(torch.float16)
    V = torch.randn(2, 8, 2, 16).to(torch.float16)
    Kp, Vp, bt, ln = pq_ops.contiguous_kv_to_pages(K, V, [6, 8], page_size=4)
    rKp, rVp, rbt, rln = opq.contiguous_kv_to_pages(K, V, [6, 8], page_size=4)
    assert torch.equal(Kp, rKp) and torch.equal(Vp, rVp) and torch.equal(bt, rbt) and torch.equal(ln, rln)
    assert bt.tolist() == [[0, 1], [2, 3]]
    K2, V2 = pq_ops.pages_to_contiguous_kv(Kp, Vp, bt, ln)
    rK2, rV2 = opq.pages_to_contiguous_kv(rKp, rVp, rbt, rln)
    assert torch.equal(K2, rK2) and torch.equal(V2, rV2)
    assert torch.equal(K2[0, :6], K[0, :6]) and float(K2[0, 6:].abs().max()) == 0.0
    _, _, bt_short, _ = pq_ops.contiguous_kv_to_pages(K, V, [3, 8], page_size=4)
    assert bt_short.tolist() == [[0, -1], [2, 3]]


def test_paged_attention_validation_errors():
    cache = pq_ops.PagedQuantizedKVCache(
        k_pages_q=torch.zeros(4, 4, 2, 16, dtype=torch.uint8), v_pages_q=torch.zeros(4, 4, 2, 16, dtype=torch.uint8),
        k_scales=torch.ones(4, 4, 2, 1, dtype=torch.float16), v_scales=torch.ones(4, 4, 2, 1, dtype=torch.float16),
        block_table=torch.arange(4, dtype=torch.int32).reshape(1, 4), lengths=torch.tensor([16], dtype=torch.int32),
        bits=8, page_size=4, group_size=32, original_page_shape=(4, 4, 2, 16))
    q = torch.randn(1, 1, 4, 16).to(torch.float16)
    fn = pq_ops.paged_quantized_kv_gqa_decode_attention
    with pytest.raises(cabi.ReferenceBackendUnavailable):
        fn(q, cache)                       # default backend is "reference", as in the reference
    with pytest.raises(ValueError, match="requires bits=4"):
        fn(q, cache, backend="metal_q4")
    with pytest.raises(ValueError, match="backend must be one of"):
        fn(q, cache, backend="metal")
    with pytest.raises(ValueError, match=r"\[B,1,Hq,D\]"):
        fn(q[:, 0], cache, backend="metal_q8")
    with pytest.raises(ValueError, match="batch mismatch"):
        fn(torch.cat([q, q]), cache, backend="metal_q8")
    with pytest.raises(ValueError, match="head_dim mismatch"):
        fn(q[..., :8], cache, backend="metal_q8")
    with pytest.raises(ValueError, match="divisible"):
        fn(torch.randn(1, 1, 3, 16).to(torch.float16), cache, backend="metal_q8")
    with pytest.raises(cabi.B200QError, match="no CPU route"):
        fn(q, cache, backend="metal_q8")
    no_shape = dataclasses.replace(cache, original_page_shape=None)
    with pytest.raises(ValueError, match="original_page_shape is required"):
        fn(q, no_shape, backend="metal_q8")


def test_contiguous_quantized_cache_host_logic():
    C = qkv_ops.QuantizedKVCacheConfig
    assert dataclasses.asdict(C()) == dict(bits=8, group_size=32, symmetric=True, with_zeros=False,
                                           scale_dtype="float16", layout="contiguous")
    with pytest.raises(ValueError):
        C(bits=5).validate()
    with pytest.raises(ValueError):
        C(group_size=0).validate()
    with pytest.raises(NotImplementedError):
        C(symmetric=False).validate()
    with pytest.raises(NotImplementedError):
        C(with_zeros=True).validate()
    with pytest.raises(NotImplementedError):
        C(layout="paged").validate()
    # container checks on caches quantised by the oracle (the quantiser is a CUDA kernel: no CPU route)
    torch.manual_seed(3)
    K = torch.randn(2, 6, 2, 40).to(torch.float16)
    V = torch.randn(2, 6, 2, 40).to(torch.float16)
    with pytest.raises(cabi.B200QError, match="no CPU route"):
        qkv_ops.quantize_kv_cache(K, V, C(bits=8, group_size=32), lengths=[6, 2])
    for bits in (8, 4):
        ref = ocq.quantize_kv_cache(K, V, bits=bits, group_size=32, lengths=[6, 2])
        cache = qkv_ops.QuantizedKVCache(**{f.name: getattr(ref, f.name) for f in dataclasses.fields(ref)})
        dp = 20 if bits == 4 else 40
        assert cache.shapes() == {"k_q": (2, 6, 2, dp), "v_q": (2, 6, 2, dp), "k_scales": (2, 6, 2, 2),
                                  "v_scales": (2, 6, 2, 2), "original": (2, 6, 2, 40)}
        assert cache.memory_bytes() == 2 * 2 * 6 * 2 * dp + 2 * 2 * 6 * 2 * 2 * 2
        assert cache.compression_ratio() == (2 * 2 * 6 * 2 * 40 * 2) / cache.memory_bytes()
        cache.validate()
    with pytest.raises(ValueError, match="must match"):
        qkv_ops.quantize_kv_cache(K, V[:1], C())
    with pytest.raises(ValueError, match="4-D"):
        qkv_ops.quantize_kv_cache(K[0], V[0], C())
    with pytest.raises(ValueError, match="positions must be in"):
        qkv_ops.quantize_kv_cache(K, V, C(), lengths=[7, 1])

    q = torch.randn(2, 1, 4, 40).to(torch.float16)
    fn = qkv_ops.quantized_kv_gqa_decode_attention
    with pytest.raises(cabi.ReferenceBackendUnavailable):
        fn(q, cache)                       # default backend is "reference", as in the reference
    with pytest.raises(ValueError, match="requires bits=8"):
        fn(q, cache, backend="metal_q8")
    with pytest.raises(ValueError, match="backend must be one of"):
        fn(q, cache, backend="metal")
    with pytest.raises(ValueError, match=r"\[B,1,Hq,D\]"):
        fn(q[:, 0], cache, backend="metal_q4")
    with pytest.raises(ValueError, match="batch mismatch"):
        fn(q[:1], cache, backend="metal_q4")
    with pytest.raises(ValueError, match="head_dim mismatch"):
        fn(q[..., :8], cache, backend="metal_q4")
    with pytest.raises(ValueError, match="positions must be in"):
        fn(q, cache, [7, 1], backend="metal_q4")
    with pytest.raises(cabi.B200QError, match="no CPU route"):
        fn(q, cache, backend="metal_q4")
    P = sparse_ops.SparseAttentionPattern
    with pytest.raises(TypeError, match="SparseAttentionPattern"):
        qkv_ops.quantized_kv_sparse_gqa_decode_attention(q, cache, None, None)
    with pytest.raises(cabi.ReferenceBackendUnavailable):
        qkv_ops.quantized_kv_sparse_gqa_decode_attention(q, cache, None, P("dense"))
    with pytest.raises(NotImplementedError):
        qkv_ops.quantized_kv_sparse_gqa_decode_attention(q, cache, None, P("dense"), backend="metal_q4")
    with pytest.raises(cabi.B200QError, match="no CPU route"):      # block_sparse is served by the CUDA backend too
        qkv_ops.quantized_kv_sparse_gqa_decode_attention(q, cache, None, P("block_sparse", block_size=4, block_mask=[[1]]),
                                                         backend="cuda")
    with pytest.raises(ValueError, match="block_sparse requires block_mask"):
        qkv_ops.quantized_kv_sparse_gqa_decode_attention(q, cache, None, P("block_sparse", block_size=4), backend="cuda")
    with pytest.raises(ValueError, match="decode_block_mask"):
        sparse_ops.decode_window(P("block_sparse", block_size=4, block_mask=[[1]]))
    bm, bs = sparse_ops.decode_block_mask(P("block_sparse", block_size=4, block_mask=[[1, 0], [2, 1]]), "cpu")
    assert bs == 4 and bm.dtype == torch.uint8 and bm.tolist() == [[1, 0], [1, 1]]
    with pytest.raises(ValueError, match="window_size > 0"):
        qkv_ops.quantized_kv_sparse_gqa_decode_attention(q, cache, None, P("sliding_window"), backend="cuda")
    with pytest.raises(cabi.B200QError, match="no CPU route"):
        qkv_ops.quantized_kv_sparse_gqa_decode_attention(q, cache, None, P("sliding_window", window_size=3), backend="cuda")
    assert sparse_ops.decode_window(P("dense")) == (0, 0)
    assert sparse_ops.decode_window(P("sliding_window", window_size=5, sink_tokens=2)) == (0, 5)
    assert sparse_ops.decode_window(P("sliding_window_sink", window_size=5, sink_tokens=2)) == (2, 5)
    with pytest.raises(ValueError, match="sink_tokens"):
        P("sliding_window_sink", window_size=5, sink_tokens=-1).validate()
    with pytest.raises(ValueError, match="pattern must be one of"):
        P("strided").validate()
    # the (sink, window) pair is the decode row of the reference's mask builder
    for L in (1, 2, 7, 16, 33):
        for W in (1, 3, 16, 40):
            for S in (0, 1, 5):
                pos = torch.arange(L)
                assert torch.equal(osparse.decode_row(L, "sliding_window_sink", window_size=W, sink_tokens=S),
                                   (pos < S) | (pos >= L - W))
                assert torch.equal(osparse.decode_row(L, "sliding_window", window_size=W, sink_tokens=S), pos >= L - W)
        assert bool(osparse.decode_row(L, "dense").all())
    # the paged view shares the buffers: 16-token pages when MAX_S allows it, else one page per sequence
    view = qkv_ops.as_paged_view(cache, torch.tensor([6, 2], dtype=torch.int32))
    assert view.page_size == 6 and view.block_table.tolist() == [[0], [1]] and view.k_pages_q.data_ptr() == cache.k_q.data_ptr()
    bref = ocq.quantize_kv_cache(torch.zeros(2, 32, 1, 16), torch.zeros(2, 32, 1, 16), bits=8, group_size=32)
    big = qkv_ops.QuantizedKVCache(**{f.name: getattr(bref, f.name) for f in dataclasses.fields(bref)})
    view = qkv_ops.as_paged_view(big, torch.tensor([32, 32], dtype=torch.int32))
    assert view.page_size == 16 and view.block_table.tolist() == [[0, 1], [2, 3]] and view.original_page_shape == (4, 16, 1, 16)


def test_block_table_lookup_host_checks():
    bt = torch.arange(8, dtype=torch.int32).reshape(2, 4)
    with pytest.raises(ValueError, match="PAGE_SIZE must be positive"):
        pkv_ops.block_table_lookup(bt, 0, 0)
    with pytest.raises(ValueError, match="positions must be in"):
        pkv_ops.block_table_lookup(bt, 16, 4)
    with pytest.raises(ValueError, match="scalar or shape"):
        pkv_ops.block_table_lookup(bt, [1, 2, 3], 4)
    with pytest.raises(ValueError, match="2-D"):
        pkv_ops.block_table_lookup(bt[0], 1, 4)
    assert pkv_ops.make_identity_block_table(2, 32, 8).tolist() == [[0, 1, 2, 3], [4, 5, 6, 7]]


def test_synth_generators_are_seeded_and_affine_formula_holds():
    a = synth.quantized_weight(16, 128, 4, 64, seed=1001)
    b = synth.quantized_weight(16, 128, 4, 64, seed=1001)
    assert all(torch.equal(u, v) for u, v in zip(a, b))
    packed, scales, zeros = a
    assert packed.shape == (16, 64) and scales.shape == (16, 2) and scales.dtype == torch.float16
    # (code - zero) * scale reproduces the weights to half a step
    w = synth._randn((16, 128), 1001, "cpu", std=0.02)
    deq = oq.reference_dequant_q4(packed, scales, zeros, group_size=64).float()
    step = scales.float().repeat_interleave(64, dim=1)
    assert bool(((deq - w).abs() <= 0.56 * step + 1e-4).all())
    case = synth.paged_kv_case(4, 2, 32, 16, 64, 5, 200, 4, 32, seed=7)
    used = case["block_table"][case["block_table"] >= 0]
    assert used.numel() == used.unique().numel()          # pages are not shared between sequences
    assert int(((case["lengths"] + 15) // 16).sum()) == used.numel()


def test_c_abi_rejects_bad_arguments_before_touching_a_device():
    """Argument checks of the C entry points run on the host: null pointers and impossible sizes come back as
    error codes (never a crash), also on a machine without a GPU."""
    import ctypes
    lib = cabi.load()
    bad = -1            # B200Q_ERR_BAD_ARG
    unsupported = -2    # B200Q_ERR_UNSUPPORTED
    assert lib.b200q_qmatvec(4, None, None, None, None, None, None, 1, 16, 64, 32, 0, 0, None) == bad
    assert lib.b200q_qmatvec(5, 1, 1, 1, None, None, 1, 1, 16, 64, 32, 0, 0, None) == bad          # bits
    assert lib.b200q_dequant(4, None, None, None, None, 4, 64, 32, 0, 0, None) == bad
    assert lib.b200q_paged_gqa_decode_static(4, None, None, None, None, None, None, None, None, 0, 32, 8, 128, 16, 1, 1, 32,
                                             1.0, 0, 0, None) == bad
    # tensor-parallel exchange: world size, rank and row size are validated
    ptrs = (ctypes.c_void_p * 2)(16, 32)
    assert lib.b200q_peer_allgather(None, ptrs, ptrs, 16, 0, 2, 1, 32, None) == bad
    assert lib.b200q_peer_allgather(16, ptrs, ptrs, 16, 2, 2, 1, 32, None) == bad                 # rank >= world
    assert lib.b200q_peer_allgather(16, ptrs, ptrs, 16, 0, 9, 1, 32, None) == bad                 # world > 8
    assert lib.b200q_peer_allgather(16, ptrs, ptrs, 16, 0, 2, 1, 24, None) == unsupported         # rows of 24 bytes
    assert b"scratch" in lib.b200q_strerror(-6)


def test_window_page_walk_covers_exactly_the_attended_positions():
    """The rule by which the split-KV attention kernel lists the pages of a sequence under a sliding window
    (csrc/paged_attn.cu: seq_pages, page_mask16), restated on the host: the listed pages are strictly increasing,
    each holds at least one attended slot, and the union of their slot masks is the decode row of the reference's
    mask builder."""
    P = 16

    def seq_pages(L, sink, window):
        n_all = (L + P - 1) // P
        if window <= 0 or L <= 0:
            return n_all, n_all, n_all
        lo = max(0, L - window)
        sink_pages = (min(sink, lo) + P - 1) // P
        first_recent = max(sink_pages, lo // P)
        return sink_pages + n_all - first_recent, sink_pages, first_recent

    def page_mask(pg, L, sink, window):
        valid = min(16, L - pg * 16)
        m = (1 << max(valid, 0)) - 1
        if window > 0:
            lo_t = max(0, L - window) - pg * 16
            sink_t = sink - pg * 16
            recent = 0xFFFF if lo_t <= 0 else (0 if lo_t >= 16 else (0xFFFF << lo_t) & 0xFFFF)
            sinks = 0 if sink_t <= 0 else (0xFFFF if sink_t >= 16 else (1 << sink_t) - 1)
            m &= recent | sinks
        return m

    for L in (1, 2, 15, 16, 17, 31, 32, 33, 100, 257):
        for sink in (0, 1, 4, 16, 20, 300):
            for window in (1, 5, 16, 17, 64, 1000):
                n, sink_pages, first_recent = seq_pages(L, sink, window)
                pages = [i if i < sink_pages else first_recent + (i - sink_pages) for i in range(n)]
                assert pages == sorted(set(pages)) and all(0 <= pg < (L + P - 1) // P for pg in pages)
                seen = torch.zeros(L, dtype=torch.bool)
                for pg in pages:
                    m = page_mask(pg, L, sink, window)
                    assert m != 0, (L, sink, window, pg)
                    for t in range(16):
                        if (m >> t) & 1:
                            seen[pg * 16 + t] = True
                want = osparse.decode_row(L, "sliding_window_sink" if sink else "sliding_window", window_size=window,
                                          sink_tokens=sink)
                assert torch.equal(seen, want), (L, sink, window)


def test_header_lists_every_tuning_key_the_library_reads():
    """b200q_set_tuning takes free-form keys; the list in include/b200q.h must name each key the sources read."""
    import re
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    header = (root / "include" / "b200q.h").read_text()
    keys = set()
    for src in (root / "mlx-metal-kernels_b200" / "csrc").glob("*.cu*"):
        keys |= set(re.findall(r'tuning_get\("([a-z0-9_.]+)"\)', src.read_text()))
    assert len(keys) >= 20
    missing = sorted(k for k in keys if f'"{k}"' not in header)
    assert not missing, missing


def test_new_entry_points_validate_their_arguments_without_a_device():
    """Argument checks of the entry points added for block-sparse decode, fp16 pages, the KV quantiser, the packet
    exchange and the wait self-test return before anything is launched, so they can be exercised without a GPU."""
    lib = cabi.load()
    BAD_ARG, UNSUPPORTED = -1, -2
    # fp16 paged decode: null pointers, heads that do not divide, head dim above 128
    assert lib.b200q_paged_fp16_gqa_decode(None, None, None, None, None, None, None, 0, 1, 4, 2, 64, 16, 8, 4, 0.125, 0, None) == BAD_ARG
    assert lib.b200q_paged_fp16_gqa_workspace_bytes(0, 4, 2, 4) == 0
    assert lib.b200q_paged_fp16_gqa_workspace_bytes(1, 4, 2, 1) == 0           # one CTA per head suffices: no scratch
    # block-sparse decode: a null mask or a non-positive block size
    args = [8] + [None] * 9 + [0]
    assert lib.b200q_paged_gqa_decode_block_sparse(*args, None, 1, 1, 16, None, 1, 4, 2, 128, 16, 8, 4, 32, 0.1, 0, 0, None) == BAD_ARG
    # packet form of a slot that was never registered; wait self-test outside its range
    assert lib.b200q_tp_set_packets(9, 1) == BAD_ARG
    assert lib.b200q_tp_set_packets(99, 1) == BAD_ARG
    assert lib.b200q_wait_expiry_selftest(0, None, None) == BAD_ARG
    assert lib.b200q_wait_expiry_selftest(1 << 17, None, None) == BAD_ARG
    # KV quantiser: null pointers
    assert lib.b200q_quantize_kv(8, None, None, None, 4, 128, 32, 0, None) == BAD_ARG
    assert UNSUPPORTED != BAD_ARG
