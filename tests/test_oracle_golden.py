"""Pins the CPU oracle against outputs of code the reference itself ships.

Sources of the fixtures (tests/golden/make_golden.py): the reference's numpy quantiser /
dequantiser (models/quantize_weights.py) and its Metal kernel bodies compiled as C++.
"""
import numpy as np
import pytest
import torch

from oracle import elementwise_ops, paged_kv_ops, paged_quantized_kv_ops as pq, quant_ops as oq
from oracle import quantized_kv_cache_ops as oc


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("tag", ["a", "b"])
def test_dequant_matches_reference_numpy_dequantizer(golden, bits, tag):
    key = f"np_q{bits}{tag}"
    G = int(golden[f"{key}_G"])
    codes, scales, zeros = t(golden[f"{key}_codes"]), t(golden[f"{key}_scales"]), t(golden[f"{key}_zeros"])
    fn = oq.reference_dequant_q4 if bits == 4 else oq.reference_dequant_q8
    sym_zero = torch.full(scales.shape, 8.0 if bits == 4 else 128.0)
    for z, want in ((sym_zero, golden[f"{key}_deq_sym"]), (zeros, golden[f"{key}_deq_zero"])):
        for dt in (torch.float16, torch.bfloat16):
            got = fn(codes, scales, z, group_size=G, out_dtype=dt)
            # the numpy reference stops at fp32; the MLX path adds one round-to-nearest cast
            assert torch.equal(got, t(want).to(dt))


def test_pack_matches_reference_numpy_packer(golden):
    codes = t(golden["np_pack_codes"])
    packed = oq.pack_q4(codes)
    assert torch.equal(packed, t(golden["np_pack_packed"]))
    assert torch.equal(oq.unpack_q4_reference(packed, K=codes.shape[1]), codes)


@pytest.mark.parametrize("bits", [4, 8])
def test_symmetric_weight_quantizer_fixture_roundtrip(golden, bits):
    # codes produced by the reference quantiser dequantise to within half a step of the weights
    key = f"np_q{bits}a"
    w = golden[f"{key}_w"]
    deq = golden[f"{key}_deq_sym"]
    G = int(golden[f"{key}_G"])
    step = np.repeat(golden[f"{key}_scales"].astype(np.float32), G, axis=1)[:, : w.shape[1]]
    # half a quantisation step, plus the fp16 rounding of the stored scale times the largest code
    assert np.all(np.abs(deq - w) <= 0.5 * step + 128 * step * 2.0 ** -11 + 1e-7)


@pytest.mark.parametrize("bits", [4, 8])
def test_dequant_matches_metal_kernel_body(golden, bits):
    key = f"mtl_q{bits}"
    codes, scales, zeros = t(golden[f"{key}_codes"]), t(golden[f"{key}_scales"]), t(golden[f"{key}_zeros"])
    fn = oq.reference_dequant_q4 if bits == 4 else oq.reference_dequant_q8
    assert torch.equal(fn(codes, scales, zeros, group_size=32), t(golden[f"{key}_deq_zero"]))
    assert torch.equal(fn(codes, scales, None, group_size=32), t(golden[f"{key}_deq_nozero"]))


@pytest.mark.parametrize("bits", [4, 8])
def test_matvec_matches_metal_kernel_body(golden, bits):
    # The Metal kernel keeps W in fp32 and sums serially; the MLX path rounds W to fp16 first.
    # They agree to fp16 weight-rounding error, which is what this bound states.
    key = f"mtl_q{bits}"
    codes, zeros, x = t(golden[f"{key}_codes"]), t(golden[f"{key}_zeros"]), t(golden[f"{key}_x"])
    scales = t(golden[f"{key}_scales"]) * 0.01
    fn = oq.reference_q4_matvec_decode if bits == 4 else oq.reference_q8_matvec_decode
    for z, want in ((zeros, golden[f"{key}_matvec_zero"]), (None, golden[f"{key}_matvec_nozero"])):
        got = fn(x, codes, scales, z, group_size=32).float()
        want = t(want).float()
        assert float((got - want).norm() / want.norm()) < 1.5e-3


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("tag", ["gqa", "mqa", "d16"])
def test_paged_attention_matches_metal_kernel_body(golden, bits, tag):
    key = f"mtl_attn_q{bits}_{tag}"
    g = {n: golden[f"{key}_{n}"] for n in ("q", "kq", "vq", "ks", "vs", "bt", "lengths", "shape", "out")}
    cache = pq.OraclePagedKV(
        k_pages_q=t(g["kq"]), v_pages_q=t(g["vq"]), k_scales=t(g["ks"]), v_scales=t(g["vs"]),
        block_table=t(g["bt"]), lengths=t(g["lengths"]), bits=bits, page_size=int(g["shape"][1]),
        group_size=32, original_page_shape=tuple(int(v) for v in g["shape"]),
    )
    got = pq.reference_paged_quantized_kv_gqa_decode_attention(t(g["q"]), cache)
    # Metal keeps dequantised K/V in fp32 and uses a streaming softmax; the MLX path rounds K/V to fp16.
    # Bound: 2e-3 absolute, widened by one fp16 ulp where the fixture's outputs exceed 1 in magnitude.
    want = t(g["out"]).float()
    assert bool(((got.float() - want).abs() <= 2e-3 + want.abs() * 2.0 ** -10).all())
    # a sequence of length 0 produces zeros
    zero_rows = np.nonzero(g["lengths"] == 0)[0]
    for b in zero_rows:
        assert float(got[b].abs().max()) == 0.0


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("tag", ["gqa", "mqa", "d16"])
def test_contiguous_attention_matches_metal_kernel_body(golden, bits, tag):
    key = f"mtl_cattn_q{bits}_{tag}"
    g = {n: golden[f"{key}_{n}"] for n in ("q", "kq", "vq", "ks", "vs", "lengths", "shape", "out")}
    cache = oc.OracleQuantizedKV(k_q=t(g["kq"]), v_q=t(g["vq"]), k_scales=t(g["ks"]), v_scales=t(g["vs"]), bits=bits,
                                 group_size=32, original_shape=tuple(int(v) for v in g["shape"]))
    got = oc.reference_quantized_kv_gqa_decode_attention(t(g["q"]), cache, t(g["lengths"]))
    # same bound as the paged pin: Metal keeps dequantised K/V in fp32, the MLX path rounds them to fp16
    want = t(g["out"]).float()
    assert bool(((got.float() - want).abs() <= 2e-3 + want.abs() * 2.0 ** -10).all())


def test_contiguous_cache_quantiser_masks_past_the_length_and_round_trips():
    gen = torch.Generator().manual_seed(5)
    K = torch.randn((2, 9, 2, 48), generator=gen).to(torch.float16)
    V = torch.randn((2, 9, 2, 48), generator=gen).to(torch.float16)
    for bits, step in ((8, 127.0), (4, 7.0)):
        cache = oc.quantize_kv_cache(K, V, bits=bits, group_size=32, lengths=[9, 4])
        assert cache.k_q.shape == (2, 9, 2, 48 if bits == 8 else 24) and cache.k_scales.shape == (2, 9, 2, 2)
        assert int(cache.k_q[1, 4:].max()) == 0 and float(cache.v_scales[1, 4:].abs().max()) == 0.0
        Kd, Vd = oc.dequantize_kv_cache(cache)
        # half a quantisation step of the group's scale, plus the fp16 roundings of scale and result
        bound = K[0].float().abs().amax() / step * 0.5 * 1.01 + 2e-3
        assert float((Kd[0].float() - K[0].float()).abs().max()) <= float(bound)
        assert float(Kd[1, 4:].abs().max()) == 0.0      # code 0 with scale 0 dequantises to 0
        # the same cache through the paged quantiser (one page per sequence) gives the same codes where valid
        paged = pq.quantize_kv_pages(K, V, None, None, bits=bits, page_size=9, group_size=32)
        assert torch.equal(paged.k_pages_q[0], cache.k_q[0]) and torch.equal(paged.v_scales[0], cache.v_scales[0])


def test_swiglu_matches_metal_kernel_body(golden):
    got = elementwise_ops.reference_swiglu(t(golden["mtl_swiglu_gate"]), t(golden["mtl_swiglu_up"]))
    want = t(golden["mtl_swiglu_out"])
    # expf implementations differ in the last bit; allow one fp16 ulp
    assert float((got.float() - want.float()).abs().max()) <= float(want.float().abs().max()) * 2 ** -10


def test_block_table_lookup_matches_metal_kernel_body(golden):
    pages, offsets = paged_kv_ops.reference_block_table_lookup(t(golden["mtl_btl_table"]), t(golden["mtl_btl_pos"]), 8)
    assert torch.equal(pages, t(golden["mtl_btl_pages"]))
    assert torch.equal(offsets, t(golden["mtl_btl_offsets"]))


def test_sparse_mask_rule_known_answers():
    """The mask rows the reference's own tests expect of build_sparse_attention_mask
    (tests/test_sparse_attention_reference.py:15-39): sliding window, window + sinks, overlap of sinks and window,
    and the block_sparse rule on a 2x2 block mask."""
    from oracle.sparse_attention_ops import build_sparse_attention_mask, decode_row
    rows = build_sparse_attention_mask(4, 6, "sliding_window", window_size=3, start_position=2).tolist()
    assert rows[0] == [True, True, True, False, False, False]
    assert rows[1] == [False, True, True, True, False, False]
    assert rows[3] == [False, False, False, True, True, True]
    row = build_sparse_attention_mask(1, 6, "sliding_window_sink", window_size=3, sink_tokens=2, start_position=4)
    assert row.tolist()[0] == [True, True, True, True, True, False]
    row = build_sparse_attention_mask(1, 5, "sliding_window_sink", window_size=4, sink_tokens=2, start_position=1)
    assert row.tolist()[0] == [True, True, False, False, False]
    block_mask = [[True, False], [True, True]]
    m = build_sparse_attention_mask(4, 4, "block_sparse", block_size=2, block_mask=block_mask)
    assert tuple(m.shape) == (4, 4)
    assert m.tolist() == [[True, False, False, False], [True, True, False, False],
                          [True, True, True, False], [True, True, True, True]]
    # the decode row is the last row of the square mask
    assert decode_row(4, "block_sparse", block_size=2, block_mask=block_mask).tolist() == m.tolist()[3]
    assert decode_row(6, "sliding_window_sink", window_size=3, sink_tokens=2).tolist() == \
        build_sparse_attention_mask(6, 6, "sliding_window_sink", window_size=3, sink_tokens=2).tolist()[5]


def _ulp16(a):
    """Spacing of fp16 at |a| (normal range)."""
    a = a.float().abs().clamp_min(2.0 ** -14)
    return torch.exp2(torch.floor(torch.log2(a)) - 10)


def test_residual_add_and_swiglu_match_metal_kernel_bodies(golden):
    x, res = t(golden["tg_norm_x"]), t(golden["tg_norm_res"])
    assert torch.equal(elementwise_ops.reference_residual_add(x, res), t(golden["tg_residual_add"]))     # one rounding
    got = elementwise_ops.reference_swiglu(x * 3, res)
    want = t(golden["tg_swiglu"])
    assert bool(((got.float() - want.float()).abs() <= _ulp16(want)).all())      # expf differs in its last bit


def test_rms_norm_matches_metal_kernel_bodies(golden):
    """rms_norm.metal and rmsnorm_residual.metal on the threadgroup emulator.  The sum of squares is taken in another
    order (strided partials, simd_sum, whose order Metal leaves open) and rmsnorm_residual.metal normalises the unrounded
    x + residual where the MLX reference rounds z first, so outputs may differ by one fp16 step; z is exact."""
    x, res, w = t(golden["tg_norm_x"]), t(golden["tg_norm_res"]), t(golden["tg_norm_w"])
    got = elementwise_ops.reference_rms_norm(x, w, eps=1e-5)
    want = t(golden["tg_rms_norm"])
    diff = (got.float() - want.float()).abs()
    assert bool((diff <= _ulp16(want)).all()) and float((diff > 0).float().mean()) < 0.02
    y, z = elementwise_ops.reference_rmsnorm_residual(x, res, w, eps=1e-5, return_residual=True)
    assert torch.equal(z, t(golden["tg_rmsnorm_residual_z"]))
    want_y = t(golden["tg_rmsnorm_residual_y"])
    diff = (y.float() - want_y.float()).abs()
    assert bool((diff <= _ulp16(want_y)).all()) and float((diff > 0).float().mean()) < 0.25


@pytest.mark.parametrize("bits", [4, 8])
def test_tiled_and_parallel_matvec_match_metal_kernel_bodies(golden, bits):
    """The ``metal_parallel`` and ``metal_tiled`` bodies (threadgroup tree reductions, fp32 weights) against the
    oracle's matvec (fp16-rounded W, fp32 matmul): same function up to the fp16 weight rounding, as for the serial
    body; N = 10 leaves a ragged last tile."""
    key = f"tg_q{bits}"
    codes, scales, zeros, x = (t(golden[f"{key}_{n}"]) for n in ("codes", "scales", "zeros", "x"))
    fn = oq.reference_q4_matvec_decode if bits == 4 else oq.reference_q8_matvec_decode
    for z, names in ((zeros, ("parallel", "tiled")), (None, ("tiled_nozero",))):
        got = fn(x, codes, scales, z, group_size=32).float()
        for name in names:
            want = t(golden[f"{key}_{name}"]).float()
            assert float((got - want).norm() / want.norm()) < 1.5e-3, name
    # the two Metal bodies themselves agree to summation order
    a, b = t(golden[f"{key}_parallel"]).float(), t(golden[f"{key}_tiled"]).float()
    assert float((a - b).norm() / b.norm()) < 1e-3


@pytest.mark.parametrize("bits", [4, 8])
def test_gate_up_matches_metal_kernel_body(golden, bits):
    key = f"tg_q{bits}"
    codes, codes2, scales, scales2, zeros, x = (t(golden[f"{key}_{n}"]) for n in
                                                ("codes", "codes2", "scales", "scales2", "zeros", "x"))
    gate, up = oq.reference_gate_up_matvec(x, codes, codes2, scales, scales2, zeros, None, bits=bits, group_size=32)
    for got, name in ((gate, "gate"), (up, "up")):
        want = t(golden[f"{key}_{name}"]).float()
        assert float((got.float().reshape(want.shape) - want).norm() / want.norm()) < 1.5e-3, name
