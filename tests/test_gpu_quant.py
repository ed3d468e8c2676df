"""GPU parity: dequant (bit-exact) and the q4/q8 matvec family against the CPU oracle.

Tolerances: dequant bitwise; matvec rel-L2 <= 1e-3 for fp16 activations with fp32 accumulation.
bf16 activations on the tensor-core path are held to 6e-3: the oracle rounds the dequantised
weights to bf16 (8 significant bits) while the kernel keeps fp16 weights, so the two differ by
bf16 weight rounding (about 1.1e-3 relative) - the reference's own bf16 bound is 5e-2.
"""
import numpy as np
import pytest
import torch

from helpers import cabi, quant_ops, random_quant_case, rel_l2, synth, to_dev
from oracle import quant_ops as oq

pytestmark = pytest.mark.gpu

TOL_F16 = 1e-3
TOL_BF16_TC = 6e-3


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,K,G", [(4, 64, 32), (8, 96, 16), (5, 80, 32), (3, 50, 16), (64, 4096, 64)])
@pytest.mark.parametrize("zeros", ["float", None])
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("scale_dtype", [torch.float32, torch.float16])
def test_dequant_bit_exact(cuda, bits, M, K, G, zeros, out_dtype, scale_dtype):
    if bits == 4 and K % 2:
        pytest.skip("q4 rows hold an even number of codes")
    codes, scales, z = random_quant_case(bits, M, K, G, seed=M * K + bits, zeros=zeros, scale_dtype=scale_dtype)
    ref_fn = oq.reference_dequant_q4 if bits == 4 else oq.reference_dequant_q8
    fn = quant_ops.dequant_q4 if bits == 4 else quant_ops.dequant_q8
    want = ref_fn(codes, scales, z, group_size=G, out_dtype=out_dtype)
    got = fn(*to_dev(cuda, codes, scales, z), group_size=G, out_dtype=out_dtype, backend="cuda")
    assert got.dtype == out_dtype and got.shape == want.shape
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))
    # the generic entry point routes by bits
    got2 = quant_ops.groupwise_dequant(*to_dev(cuda, codes, scales, z), bits=bits, group_size=G, out_dtype=out_dtype)
    assert torch.equal(got2, got)


@pytest.mark.parametrize("bits", [4, 8])
def test_dequant_matches_reference_fixtures(cuda, golden, bits):
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    for tag in ("a", "b"):
        key = f"np_q{bits}{tag}"
        G = int(golden[f"{key}_G"])
        fn = quant_ops.dequant_q4 if bits == 4 else quant_ops.dequant_q8
        got = fn(*to_dev(cuda, t(golden[f"{key}_codes"]), t(golden[f"{key}_scales"]), t(golden[f"{key}_zeros"])),
                 group_size=G)
        assert torch.equal(got.cpu(), t(golden[f"{key}_deq_zero"]).to(torch.float16))
    key = f"mtl_q{bits}"
    fn = quant_ops.dequant_q4 if bits == 4 else quant_ops.dequant_q8
    got = fn(*to_dev(cuda, t(golden[f"{key}_codes"]), t(golden[f"{key}_scales"]), t(golden[f"{key}_zeros"])), group_size=32)
    assert torch.equal(got.cpu(), t(golden[f"{key}_deq_zero"]))


def test_dequant_full_size_c1_weights(cuda):
    packed, scales, zeros = synth.quantized_weight(4096, 4096, 4, 64, seed=1001)
    want = oq.reference_dequant_q4(packed, scales, zeros, group_size=64)
    got = quant_ops.dequant_q4(*to_dev(cuda, packed, scales, zeros), group_size=64)
    assert torch.equal(got.cpu(), want)


# (B, K, N, G, zeros, dtype): the reference's matvec test matrix (tests/test_quant_matvec*.py) ...
REF_CASES = [
    (1, 64, 32, 32, None, torch.float16),
    (1, 64, 32, 32, "float", torch.bfloat16),
    (2, 128, 64, 32, None, torch.float16),
    (2, 128, 64, 32, "float", torch.bfloat16),
    (1, 96, 48, 16, "float", torch.float16),
    (1, 96, 50, 16, None, torch.float16),
    (2, 96, 50, 16, "float", torch.bfloat16),
]
# ... and shapes that exercise the tensor-core path (K % 128 == 0, G % 32 == 0)
FAST_CASES = [
    (1, 128, 16, 32, "float", torch.float16),
    (1, 256, 50, 64, "float", torch.float16),
    (3, 512, 200, 128, None, torch.float16),
    (8, 1024, 333, 64, "float", torch.float16),
    (5, 2048, 1000, 32, "float", torch.float16),
    (16, 1024, 129, 64, "float", torch.float16),
    (12, 512, 64, 64, None, torch.float16),
    (20, 512, 96, 64, "float", torch.float16),
    (2, 1024, 77, 64, "float", torch.bfloat16),
]


def _matvec_case(bits, B, K, N, G, zeros, dtype, seed, scale_dtype=torch.float32):
    codes, scales, z = random_quant_case(bits, N, K, G, seed, zeros=zeros, scale_dtype=scale_dtype, scale_kind="uniform")
    x = torch.randn((B, K), generator=torch.Generator().manual_seed(seed + 1)).to(dtype)
    return x, codes, scales, z


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("case", REF_CASES + FAST_CASES)
@pytest.mark.parametrize("backend", ["auto", "metal_parallel", "metal_tiled", "cuda"])
def test_matvec_parity(cuda, bits, case, backend):
    B, K, N, G, zeros, dtype = case
    x, codes, scales, z = _matvec_case(bits, B, K, N, G, zeros, dtype, seed=K + N + bits)
    ref = oq.reference_q4_matvec_decode if bits == 4 else oq.reference_q8_matvec_decode
    fn = quant_ops.q4_matvec_decode if bits == 4 else quant_ops.q8_matvec_decode
    want = ref(x, codes, scales, z, group_size=G)
    got = fn(*to_dev(cuda, x, codes, scales, z), group_size=G, backend=backend)
    assert got.shape == (B, N) and got.dtype == dtype
    tol = TOL_F16 if dtype == torch.float16 else TOL_BF16_TC
    assert rel_l2(got, want) <= tol


@pytest.mark.parametrize("bits", [4, 8])
def test_matvec_token_shaped_input_and_fp16_scales(cuda, bits):
    x, codes, scales, z = _matvec_case(bits, 2, 256, 40, 64, "float", torch.float16, seed=11, scale_dtype=torch.float16)
    ref = oq.reference_q4_matvec_decode if bits == 4 else oq.reference_q8_matvec_decode
    fn = quant_ops.q4_matvec_decode if bits == 4 else quant_ops.q8_matvec_decode
    want = ref(x[:, None, :], codes, scales, z, group_size=64)
    got = fn(*to_dev(cuda, x[:, None, :], codes, scales, z), group_size=64)
    assert got.shape == (2, 40)          # [B,1,K] comes back as [B,N], as in the reference
    assert rel_l2(got, want) <= TOL_F16


def test_matvec_negative_scales_like_reference_tests(cuda):
    # tests/test_quant_matvec.py draws scales from N(0,1): negative scales are legal inputs
    codes, scales, z = random_quant_case(4, 64, 256, 32, 5, zeros="float", scale_kind="normal")
    x = torch.randn(2, 256).to(torch.float16)
    want = oq.reference_q4_matvec_decode(x, codes, scales, z, group_size=32)
    got = quant_ops.q4_matvec_decode(*to_dev(cuda, x, codes, scales, z), group_size=32)
    assert rel_l2(got, want) <= TOL_F16


def test_matvec_saturates_to_finite_range(cuda):
    codes = torch.full((16, 64), 0xFF, dtype=torch.uint8)
    scales = torch.full((16, 2), 60.0)
    x = torch.full((1, 128), 100.0).to(torch.float16)
    got = quant_ops.q4_matvec_decode(*to_dev(cuda, x, codes, scales), group_size=64)
    want = oq.reference_q4_matvec_decode(x, codes, scales, group_size=64)
    assert torch.equal(got.cpu(), want) and float(got.max()) == 65504.0


@pytest.mark.parametrize("config", ["C1", "C2_b1", "C2_b8"])
def test_matvec_benchmark_shapes(cuda, config):
    """C1: q4 4096x4096 G64 B1 (seed 1001); C2: q8 14336x4096 G64 B1/B8 (seed 1002), fp16 scales/zeros."""
    if config == "C1":
        bits, B, N, K, seed = 4, 1, 4096, 4096, 1001
    else:
        bits, B, N, K, seed = 8, (1 if config.endswith("b1") else 8), 14336, 4096, 1002
    packed, scales, zeros = synth.quantized_weight(N, K, bits, 64, seed=seed)
    x = synth.activations((B, K), seed + 500)
    ref = oq.reference_q4_matvec_decode if bits == 4 else oq.reference_q8_matvec_decode
    fn = quant_ops.q4_matvec_decode if bits == 4 else quant_ops.q8_matvec_decode
    want = ref(x, packed, scales, zeros, group_size=64)
    dev = to_dev(cuda, x, packed, scales, zeros)
    got = fn(*dev, group_size=64)
    assert rel_l2(got, want) <= TOL_F16
    again = fn(*dev, group_size=64)
    assert torch.equal(got, again), "results must be bitwise reproducible"
    assert cabi.device_status() == 0


# (B, K, N, G, dtype) with fp16 scales / zero points, chosen to reach every branch of the tensor-core kernel's
# planning: a partial last unit (K / G not a multiple of 8), fewer groups than one unit, activations staged in
# several passes (B * K too large for shared memory), batches above 16 (split into chunks), every group size
# and column layout (1, 2, 4, 8 batch columns per group, two column tiles).
PLAN_CASES = [
    (1, 11008, 300, 64, torch.float16),
    (1, 192, 40, 64, torch.float16),
    (2, 640, 64, 32, torch.float16),
    (3, 1536, 100, 128, torch.float16),
    (4, 2560, 130, 32, torch.float16),
    (7, 4096, 96, 128, torch.float16),
    (8, 14336, 272, 64, torch.float16),
    (16, 2048, 80, 64, torch.float16),
    (32, 4096, 144, 64, torch.float16),
    (5, 1024, 48, 64, torch.bfloat16),
]


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("case", PLAN_CASES)
def test_matvec_kernel_plans(cuda, bits, case):
    B, K, N, G, dtype = case
    packed, scales, zeros = synth.quantized_weight(N, K, bits, G, seed=K + N)
    x = synth.activations((B, K), K + 7).to(dtype)
    ref = oq.reference_q4_matvec_decode if bits == 4 else oq.reference_q8_matvec_decode
    fn = quant_ops.q4_matvec_decode if bits == 4 else quant_ops.q8_matvec_decode
    want = ref(x, packed, scales, zeros, group_size=G)
    dev = to_dev(cuda, x, packed, scales, zeros)
    got = fn(*dev, group_size=G)
    assert rel_l2(got, want) <= (TOL_F16 if dtype == torch.float16 else TOL_BF16_TC)
    assert torch.equal(got, fn(*dev, group_size=G)), "results must be bitwise reproducible"
    # the general kernel is the literal reference arithmetic: both kernels must agree with each other too
    cabi.set_tuning("gemv.force_generic", 1)
    try:
        slow = fn(*dev, group_size=G)
    finally:
        cabi.set_tuning("gemv.force_generic", 0)
    assert rel_l2(got, slow) <= (TOL_F16 if dtype == torch.float16 else TOL_BF16_TC)
    assert cabi.device_status() == 0


def test_matvec_linearity_at_full_size(cuda):
    """Size-independent property: y(x1 + x2) == y(x1) + y(x2) up to fp16 rounding of the outputs."""
    packed, scales, zeros = to_dev(cuda, *synth.quantized_weight(4096, 4096, 4, 64, seed=1001))
    x1 = synth.activations((1, 4096), 1, cuda)
    x2 = synth.activations((1, 4096), 2, cuda)
    xs = (x1.float() + x2.float()).to(torch.float16)
    y1 = quant_ops.q4_matvec_decode(x1, packed, scales, zeros, group_size=64).float()
    y2 = quant_ops.q4_matvec_decode(x2, packed, scales, zeros, group_size=64).float()
    # use the exactly representable sum as the third input
    x2e = (xs.float() - x1.float()).to(torch.float16)
    y2e = quant_ops.q4_matvec_decode(x2e, packed, scales, zeros, group_size=64).float()
    ys = quant_ops.q4_matvec_decode(xs, packed, scales, zeros, group_size=64).float()
    assert rel_l2(ys, y1 + y2e) <= 2e-3
    assert float((y1 - y2).abs().max()) > 0
