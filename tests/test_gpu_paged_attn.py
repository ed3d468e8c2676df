"""GPU parity: q4/q8 paged-KV GQA decode attention and the block-table gather against the CPU
oracle.  Bound: max |out - oracle| <= 2e-3 in fp16 (K/V ~ N(0,1))."""
import dataclasses
import importlib

import numpy as np
import pytest
import torch

from helpers import cabi, pkv_ops, pq_ops, synth
from oracle import paged_kv_ops as opk, paged_quantized_kv_ops as opq

pytestmark = pytest.mark.gpu
ATOL = 2e-3


def _oracle_cache(case):
    return opq.OraclePagedKV(**{k: (v.cpu() if torch.is_tensor(v) else v) for k, v in case.items()})


def _device_cache(case, device):
    return pq_ops.PagedQuantizedKVCache(**{k: (v.to(device) if torch.is_tensor(v) else v) for k, v in case.items()})


def _case_with_lengths(lengths, Hkv, D, P, bits, G, seed, spare_pages=7):
    """K/V ~N(0,1) quantised like the reference cache; pages of each sequence drawn from one random
    permutation of the pool; block-table entries past the length are -1."""
    B = len(lengths)
    blocks = [(L + P - 1) // P for L in lengths]
    num_pages = sum(blocks) + spare_pages
    max_blocks = max(max(blocks), 1) + 1
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).to(torch.int32)
    bt = torch.full((B, max_blocks), -1, dtype=torch.int32)
    cur = 0
    for b, n in enumerate(blocks):
        bt[b, :n] = perm[cur:cur + n]
        cur += n
    shape = (num_pages, P, Hkv, D)
    kq, ks = synth.quantize_kv_symmetric(synth._randn(shape, seed + 1, "cpu"), bits, G)
    vq, vs = synth.quantize_kv_symmetric(synth._randn(shape, seed + 2, "cpu"), bits, G)
    return {"k_pages_q": kq, "v_pages_q": vq, "k_scales": ks, "v_scales": vs, "block_table": bt,
            "lengths": torch.tensor(lengths, dtype=torch.int32), "bits": bits, "page_size": P, "group_size": G,
            "original_page_shape": shape}


def _check(case, q, device, backend, atol=ATOL):
    want = opq.reference_paged_quantized_kv_gqa_decode_attention(q, _oracle_cache(case))
    got = pq_ops.paged_quantized_kv_gqa_decode_attention(q.to(device), _device_cache(case, device), backend=backend)
    assert got.shape == q.shape and got.dtype == q.dtype
    err = float((got.cpu().float() - want.float()).abs().max())
    assert err <= atol, err
    return got, want


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("B,MAX_S,Hq,Hkv,D,P", [
    (1, 16, 4, 2, 16, 4), (1, 16, 4, 1, 16, 4), (1, 16, 4, 4, 16, 4),       # tests/test_paged_quantized_kv_decode_metal.py
    (2, 16, 4, 2, 16, 4), (1, 16, 4, 2, 64, 4), (1, 16, 4, 2, 128, 4),
])
def test_reference_test_shapes_full_lengths(cuda, bits, B, MAX_S, Hq, Hkv, D, P):
    torch.manual_seed(42)
    K = torch.randn(B, MAX_S, Hkv, D).to(torch.float16)
    V = torch.randn(B, MAX_S, Hkv, D).to(torch.float16)
    Kp, Vp, bt, ln = opq.contiguous_kv_to_pages(K, V, [MAX_S] * B, page_size=P)
    oc = opq.quantize_kv_pages(Kp, Vp, bt, ln, bits=bits, page_size=P, group_size=32)
    case = {f.name: getattr(oc, f.name) for f in dataclasses.fields(oc)}
    q = torch.randn(B, 1, Hq, D).to(torch.float16)
    _check(case, q, cuda, "metal_q8" if bits == 8 else "metal_q4")
    # the quantised attention stays close to fp16 attention over the unquantised cache
    # (tests/test_paged_quantized_kv_decode_reference.py: 1.5e-1 for q8, 3e-1 for q4)
    group = Hq // Hkv
    scores = torch.einsum("bhgd,bshd->bhgs", q.float().reshape(B, Hkv, group, D), K.float()) / D ** 0.5
    dense = torch.einsum("bhgs,bshd->bhgd", torch.softmax(scores, -1), V.float()).reshape(B, 1, Hq, D)
    got = pq_ops.paged_quantized_kv_gqa_decode_attention(q.to(cuda), _device_cache(case, cuda), backend="cuda")
    assert float((got.cpu().float() - dense).abs().max()) <= (1.5e-1 if bits == 8 else 3e-1)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("B,Hq,Hkv,lengths", [
    (3, 32, 8, [100, 17, 16]),            # ragged, one sequence shorter than two pages
    (4, 32, 8, [5, 0, 250, 33]),          # shorter than a page, empty sequence
    (2, 8, 8, [64, 31]),                  # MHA
    (2, 8, 2, [47, 129]),                 # fewer kv heads than warps
    (5, 16, 4, [1, 2, 15, 16, 300]),
])
@pytest.mark.parametrize("G", [32, 64])
def test_ragged_permuted_pages_tensor_core_path(cuda, bits, B, Hq, Hkv, lengths, G):
    D, P = 128, 16
    case = _case_with_lengths(lengths, Hkv, D, P, bits, G, seed=bits * 1000 + B)
    q = synth.activations((B, 1, Hq, D), 99)
    got, want = _check(case, q, cuda, "cuda")
    for b, L in enumerate(lengths):
        if L == 0:
            assert float(got[b].abs().max()) == 0.0
    # forcing the one-warp-per-head kernel gives the same answer within the same bound
    cabi.set_tuning("attn.force_simple", 1)
    try:
        _check(case, q, cuda, "cuda")
    finally:
        cabi.set_tuning("attn.force_simple", 0)
    assert cabi.device_status() == 0


def test_unassigned_pages_inside_length_are_skipped(cuda):
    case = synth.paged_kv_case(2, 8, 128, 16, num_pages=40, min_len=100, max_len=160, bits=4, group_size=32, seed=3)
    case["block_table"][0, 2] = -1
    case["block_table"][1, 0] = -1
    q = synth.activations((2, 1, 32, 128), 4)
    _check(case, q, cuda, "cuda")


@pytest.mark.parametrize("bits", [4, 8])
def test_metal_kernel_fixtures(cuda, golden, bits):
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    for tag in ("gqa", "mqa", "d16"):
        key = f"mtl_attn_q{bits}_{tag}"
        g = {n: golden[f"{key}_{n}"] for n in ("q", "kq", "vq", "ks", "vs", "bt", "lengths", "shape", "out")}
        cache = pq_ops.PagedQuantizedKVCache(
            k_pages_q=t(g["kq"]).to(cuda), v_pages_q=t(g["vq"]).to(cuda), k_scales=t(g["ks"]).to(cuda),
            v_scales=t(g["vs"]).to(cuda), block_table=t(g["bt"]).to(cuda), lengths=t(g["lengths"]).to(cuda), bits=bits,
            page_size=int(g["shape"][1]), group_size=32, original_page_shape=tuple(int(v) for v in g["shape"]))
        got = pq_ops.paged_quantized_kv_gqa_decode_attention(t(g["q"]).to(cuda), cache, backend="cuda")
        want = t(g["out"]).float()
        assert bool(((got.cpu().float() - want).abs() <= 2e-3 + want.abs() * 2.0 ** -10).all())


@pytest.mark.parametrize("bits", [4, 8])
def test_benchmark_config_c4(cuda, bits):
    """C4: batch 16, 32 q / 8 kv heads, D 128, page 16, lengths U[1024, 8192], 9000-page pool (seed 1004)."""
    case = synth.paged_kv_case(16, 8, 128, 16, num_pages=9000, min_len=1024, max_len=8192, bits=bits, group_size=32,
                               seed=1004)
    q = synth.activations((16, 1, 32, 128), 1005)
    got, _ = _check(case, q, cuda, "cuda")
    again = pq_ops.paged_quantized_kv_gqa_decode_attention(q.to(cuda), _device_cache(case, cuda), backend="cuda")
    assert torch.equal(again, got)
    assert cabi.device_status() == 0


def test_dequantize_pages_bit_exact(cuda):
    for bits, D, G in ((8, 64, 32), (4, 64, 32), (4, 17, 16), (8, 16, 32)):
        torch.manual_seed(D)
        K = torch.randn(5, 4, 2, D).to(torch.float16)
        V = torch.randn(5, 4, 2, D).to(torch.float16)
        oc = opq.quantize_kv_pages(K, V, torch.zeros(1, 5, dtype=torch.int32), torch.tensor([20]), bits=bits,
                                   page_size=4, group_size=G)
        wK, wV = opq.dequantize_kv_pages(oc)
        dc = _device_cache({f.name: getattr(oc, f.name) for f in dataclasses.fields(oc)}, cuda)
        gK, gV = pq_ops.dequantize_kv_pages(dc)
        assert torch.equal(gK.cpu(), wK) and torch.equal(gV.cpu(), wV)
        err = pq_ops.paged_quantized_kv_error(K.to(cuda), V.to(cuda), dc)
        assert err["k_max_abs_error"] < (0.05 if bits == 8 else 0.6) and 1.0 < err["compression_ratio"] < 10.0


@pytest.mark.parametrize("B,MAX_S,P,pos", [(1, 16, 4, 3), (2, 32, 8, [2, 17])])     # tests/test_paged_kv_cache.py
def test_block_table_lookup_exact(cuda, golden, B, MAX_S, P, pos):
    bt = torch.randperm(B * (MAX_S // P)).to(torch.int32).reshape(B, MAX_S // P)
    wp, wo = opk.reference_block_table_lookup(bt, pos, P)
    gp, go = pkv_ops.block_table_lookup(bt.to(cuda), pos, P)
    assert gp.dtype == torch.int32 and torch.equal(gp.cpu(), wp) and torch.equal(go.cpu(), wo)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    fp, fo = pkv_ops.block_table_lookup(t(golden["mtl_btl_table"]).to(cuda), t(golden["mtl_btl_pos"]).to(cuda), 8)
    assert torch.equal(fp.cpu(), t(golden["mtl_btl_pages"])) and torch.equal(fo.cpu(), t(golden["mtl_btl_offsets"]))


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("sink,window", [(0, 16), (4, 32), (20, 5), (3, 1), (40, 100), (0, 4096), (16, 16)])
@pytest.mark.parametrize("Hq,Hkv,D,P", [(8, 2, 128, 16), (32, 8, 128, 16), (6, 3, 64, 8)])
def test_sliding_window_and_sinks_match_oracle(cuda, bits, sink, window, Hq, Hkv, D, P):
    """The split-KV kernel walks only the pages that hold an attended position (first shapes); other shapes run
    the general kernel with the same position filter.  Lengths straddle the window, the sink count and page
    boundaries."""
    sparse_ops = importlib.import_module("mlx_metal_kernels_b200.ops.sparse_attention_ops")
    lengths = [1, 15, 16, 17, 37, 200, 333]
    case = _case_with_lengths(lengths, Hkv, D, P, bits, 32, seed=300 + sink + window)
    q = synth.activations((len(lengths), 1, Hq, D), 71)
    want = opq.reference_paged_quantized_kv_gqa_decode_attention(q, _oracle_cache(case), window=(sink, window))
    name = "sliding_window_sink" if sink else "sliding_window"
    pattern = sparse_ops.SparseAttentionPattern(name, window_size=window, sink_tokens=sink)
    got = pq_ops.sparse_paged_quantized_kv_gqa_decode_attention(q.to(cuda), _device_cache(case, cuda), pattern)
    err = float((got.cpu().float() - want.float()).abs().max())
    assert err <= ATOL, err
    # a window that covers everything is the dense result of the same (split-KV) kernel, bit for bit: same page walk
    if window >= max(lengths):
        cabi.set_tuning("attn.cluster", -1)
        try:
            dense = pq_ops.paged_quantized_kv_gqa_decode_attention(q.to(cuda), _device_cache(case, cuda), backend="cuda")
        finally:
            cabi.set_tuning("attn.cluster", 0)
        assert torch.equal(got, dense)
    assert cabi.device_status() == 0


@pytest.mark.parametrize("bits,D,G,dtype", [(8, 32, 32, torch.float16), (4, 32, 32, torch.float16), (4, 17, 16, torch.float16),
                                            (8, 16, 32, torch.float16), (4, 128, 32, torch.bfloat16), (8, 128, 64, torch.float16),
                                            (4, 24, 3, torch.float16)])
def test_quantize_kv_pages_matches_oracle_exactly(cuda, bits, D, G, dtype):
    """quantize_kv_pages runs the CUDA quantiser (b200q_quantize_kv): codes and scales equal the oracle's bit for bit,
    including a short last group (D = 17, 16 < G), an odd group size and bf16 pages."""
    g = torch.Generator().manual_seed(bits * 100 + D)
    K = torch.randn((6, 4, 2, D), generator=g).to(dtype)
    V = (torch.randn((6, 4, 2, D), generator=g) * 3).to(dtype)
    K[0, 0, 0] = 0                                            # an all-zero group: scale 1e-8 / limit, codes at the offset
    bt = torch.arange(6, dtype=torch.int32).reshape(2, 3)
    ln = torch.tensor([12, 9], dtype=torch.int32)
    want = opq.quantize_kv_pages(K, V, bt, ln, bits=bits, page_size=4, group_size=G)
    got = pq_ops.quantize_kv_pages(K.to(cuda), V.to(cuda), bt.to(cuda), ln.to(cuda),
                                   pq_ops.PagedQuantizedKVConfig(bits=bits, page_size=4, group_size=G))
    for name in ("k_pages_q", "v_pages_q", "k_scales", "v_scales"):
        assert torch.equal(getattr(got, name).cpu(), getattr(want, name)), name
    assert got.k_scales.dtype == torch.float16


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("lengths,Hq,Hkv,G", [([4097], 32, 8, 32), ([100, 3], 32, 8, 32), ([17, 0, 5000], 32, 8, 32),
                                               ([33], 32, 8, 64), ([700, 64], 8, 2, 32), ([1], 32, 8, 32), ([16] * 6, 4, 4, 32)])
def test_cluster_kernel_matches_oracle(cuda, bits, lengths, Hq, Hkv, G):
    """The one-kernel cluster form of the attention (forced on for every shape here) against the oracle, ragged and empty
    sequences included; and it agrees with the split-KV kernels to within the bound."""
    case = _case_with_lengths(lengths, Hkv, 128, 16, bits, G, seed=77)
    q = synth.activations((len(lengths), 1, Hq, 128), 78)
    want = opq.reference_paged_quantized_kv_gqa_decode_attention(q, _oracle_cache(case))
    dcache = _device_cache(case, cuda)
    cabi.set_tuning("attn.cluster", 1)
    try:
        got = pq_ops.paged_quantized_kv_gqa_decode_attention(q.to(cuda), dcache, backend="cuda")
        cabi.set_tuning("attn.cluster", -1)
        split = pq_ops.paged_quantized_kv_gqa_decode_attention(q.to(cuda), dcache, backend="cuda")
    finally:
        cabi.set_tuning("attn.cluster", 0)
    assert float((got.cpu().float() - want.float()).abs().max()) <= ATOL
    assert float((got.float() - split.float()).abs().max()) <= ATOL
    assert cabi.device_status() == 0


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("block_size", [16, 32, 64, 8, 24])
@pytest.mark.parametrize("Hq,Hkv,D,P", [(8, 2, 128, 16), (32, 8, 128, 16), (6, 3, 64, 8)])
def test_block_sparse_decode_matches_oracle(cuda, bits, block_size, Hq, Hkv, D, P):
    """block_sparse decode: key j of a sequence of L tokens is attended iff block_mask[(L-1)//bs][j//bs].  Block sizes
    that are a multiple of the page size run the dense kernels on a compacted block table, the others (8, 24) the
    per-token test of the general kernel; both against the oracle's masked softmax."""
    sparse_ops = importlib.import_module("mlx_metal_kernels_b200.ops.sparse_attention_ops")
    from oracle.sparse_attention_ops import decode_row
    lengths = [1, 15, 16, 17, 37, 200, 333, 64]
    nblk = (max(lengths) + block_size - 1) // block_size
    g = torch.Generator().manual_seed(block_size + bits)
    mask = torch.rand((nblk, nblk), generator=g) < 0.45
    mask |= torch.eye(nblk, dtype=torch.bool)                   # every query block sees itself: no empty rows
    case = _case_with_lengths(lengths, Hkv, D, P, bits, 32, seed=500 + block_size)
    q = synth.activations((len(lengths), 1, Hq, D), 72)
    keep = lambda L: decode_row(L, "block_sparse", block_size=block_size, block_mask=mask)   # noqa: E731
    want = opq.reference_paged_quantized_kv_gqa_decode_attention(q, _oracle_cache(case), keep_fn=keep)
    pattern = sparse_ops.SparseAttentionPattern("block_sparse", block_size=block_size, block_mask=mask)
    got = pq_ops.sparse_paged_quantized_kv_gqa_decode_attention(q.to(cuda), _device_cache(case, cuda), pattern)
    err = float((got.cpu().float() - want.float()).abs().max())
    assert err <= ATOL, err
    # an all-ones mask is the dense result
    ones = sparse_ops.SparseAttentionPattern("block_sparse", block_size=block_size, block_mask=torch.ones_like(mask))
    got1 = pq_ops.sparse_paged_quantized_kv_gqa_decode_attention(q.to(cuda), _device_cache(case, cuda), ones)
    dense = opq.reference_paged_quantized_kv_gqa_decode_attention(q, _oracle_cache(case))
    assert float((got1.cpu().float() - dense.float()).abs().max()) <= ATOL
    # a row that hides every key gives zeros
    hidden = mask.clone()
    hidden[(lengths[5] - 1) // block_size] = False
    got0 = pq_ops.sparse_paged_quantized_kv_gqa_decode_attention(
        q.to(cuda), _device_cache(case, cuda),
        sparse_ops.SparseAttentionPattern("block_sparse", block_size=block_size, block_mask=hidden))
    assert float(got0[5].abs().max()) == 0.0
    assert cabi.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,P", [(4, 4, 64, 4), (8, 2, 128, 16), (32, 8, 128, 16), (6, 3, 40, 8), (16, 1, 128, 16),
                                        (12, 2, 20, 5)])
def test_fp16_paged_gqa_decode_matches_oracle(cuda, dtype, Hq, Hkv, D, P):
    """Decode attention over an unquantised paged cache (fp16 / bf16), equal and grouped heads, ragged lengths, pages
    drawn from a shuffled pool, D not a multiple of 8, unassigned block-table entries past the length."""
    gqa_ops = importlib.import_module("mlx_metal_kernels_b200.ops.gqa_ops")
    lengths = [1, 15, 16, 17, 37, 200, 777, 0]
    B = len(lengths)
    blocks = [(L + P - 1) // P for L in lengths]
    num_pages = sum(blocks) + 5
    max_blocks = max(blocks) + 1
    g = torch.Generator().manual_seed(D + Hq)
    perm = torch.randperm(num_pages, generator=g).to(torch.int32)
    bt = torch.full((B, max_blocks), -1, dtype=torch.int32)
    cur = 0
    for b, n in enumerate(blocks):
        bt[b, :n] = perm[cur:cur + n]
        cur += n
    K = torch.randn((num_pages, P, Hkv, D), generator=g).to(dtype)
    V = torch.randn((num_pages, P, Hkv, D), generator=g).to(dtype)
    q = torch.randn((B, 1, Hq, D), generator=g).to(dtype)
    ln = torch.tensor(lengths, dtype=torch.int32)
    want = opk.reference_paged_gqa_decode_attention(q, K, V, bt, ln)
    got = gqa_ops.paged_gqa_decode_attention(q.to(cuda), K.to(cuda), V.to(cuda), bt.to(cuda), ln.to(cuda))
    assert got.shape == q.shape and got.dtype == dtype
    tol = ATOL if dtype == torch.float16 else 1.6e-2             # one bf16 rounding of values up to ~2
    assert float((got.cpu().float() - want.float()).abs().max()) <= tol
    assert float(got[-1].abs().max()) == 0.0                     # no valid token: zeros
    if Hq == Hkv:
        got2 = pkv_ops.paged_decode_attention(q.to(cuda), K.to(cuda), V.to(cuda), bt.to(cuda), ln.to(cuda), backend="metal_d64")
        assert torch.equal(got2, got)
        with pytest.raises(ValueError, match=r"q must have shape \[B,1,H,D\]"):
            pkv_ops.paged_decode_attention(q[:, :, :1].to(cuda), K.to(cuda), V.to(cuda), bt.to(cuda), ln.to(cuda))


def test_fp16_paged_gqa_decode_long_context(cuda):
    """Context 4096, batch 16, 32 / 8 heads of 128: the split-over-CTAs path with its merge kernel."""
    gqa_ops = importlib.import_module("mlx_metal_kernels_b200.ops.gqa_ops")
    B, Hq, Hkv, D, P, ctx = 16, 32, 8, 128, 16, 4096
    g = torch.Generator().manual_seed(3)
    blocks = ctx // P
    num_pages = B * blocks
    bt = torch.randperm(num_pages, generator=g).to(torch.int32).reshape(B, blocks)
    K = torch.randn((num_pages, P, Hkv, D), generator=g).to(torch.float16)
    V = torch.randn((num_pages, P, Hkv, D), generator=g).to(torch.float16)
    q = torch.randn((B, 1, Hq, D), generator=g).to(torch.float16)
    ln = torch.randint(1, ctx + 1, (B,), generator=g, dtype=torch.int32)
    ln[0] = ctx
    want = opk.reference_paged_gqa_decode_attention(q, K, V, bt, ln)
    got = gqa_ops.paged_gqa_decode_attention(q.to(cuda), K.to(cuda), V.to(cuda), bt.to(cuda), ln.to(cuda))
    assert float((got.cpu().float() - want.float()).abs().max()) <= ATOL
