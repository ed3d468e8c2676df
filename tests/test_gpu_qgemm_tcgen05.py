"""GPU parity of the tcgen05 matvec kernel (weights dequantised into tensor memory) against the CPU oracle:
rel-L2 <= 1e-3 for fp16 activations with fp32 accumulation, on both of its shapes (compact: two kernels per SM;
whole SM), with and without a K split over a thread-block cluster, plain / gate-up / fused-norm entry points."""
import pytest
import torch

from helpers import cabi, mlp_ops, quant_ops, rel_l2, synth
from oracle import quant_ops as oq
from oracle.elementwise_ops import reference_swiglu

pytestmark = pytest.mark.gpu
TOL = 1e-3


@pytest.fixture
def tcgen05(cuda):
    """Routes every supported launch to the tcgen05 kernel; restores the default routing afterwards."""
    cabi.set_tuning("gemv.ts", 1)
    yield cuda
    for key in ("gemv.ts", "ts.big", "ts.split", "ts.slow_reduce", "ts.stages", "gemv.fuse_norm"):
        cabi.set_tuning(key, 0)
    assert cabi.device_status() == 0


def _ref(bits):
    return oq.reference_q4_matvec_decode if bits == 4 else oq.reference_q8_matvec_decode


def _fn(bits):
    return quant_ops.q4_matvec_decode if bits == 4 else quant_ops.q8_matvec_decode


# (bits, B, N, K, G)
SHAPES = [
    (4, 1, 128, 256, 64), (4, 3, 256, 1024, 64), (8, 1, 128, 512, 64), (8, 5, 300, 1024, 64),
    (4, 4, 1000, 2048, 32), (4, 4, 1000, 2048, 128), (8, 4, 1000, 2048, 32), (8, 4, 1000, 2048, 128),
    (4, 7, 4096, 4096, 64), (4, 16, 520, 1536, 64), (4, 17, 136, 768, 64), (4, 32, 4096, 4096, 64),
    (8, 32, 640, 2048, 64), (4, 33, 256, 512, 64), (4, 64, 384, 1024, 64),
]


@pytest.mark.parametrize("big", [-1, 1])
@pytest.mark.parametrize("case", SHAPES)
def test_matvec_shapes(tcgen05, case, big):
    bits, B, N, K, G = case
    cabi.set_tuning("ts.big", big)
    w, s, z = synth.quantized_weight(N, K, bits, G, seed=N + K + bits)
    x = synth.activations((B, K), 7)
    want = _ref(bits)(x, w, s, z, group_size=G)
    d = lambda t: t.to(tcgen05)
    got = _fn(bits)(d(x), d(w), d(s), d(z), group_size=G, backend="cuda")
    assert got.shape == (B, N)
    assert rel_l2(got, want) <= TOL
    again = _fn(bits)(d(x), d(w), d(s), d(z), group_size=G, backend="cuda")
    assert torch.equal(again, got)                      # fixed summation order: bitwise repeatable


@pytest.mark.parametrize("split,slow", [(1, 0), (2, 0), (4, 0), (4, 1), (8, 1)])
@pytest.mark.parametrize("B", [1, 12])
def test_cluster_split_k(tcgen05, split, slow, B):
    """The K range split over a cluster: partial sums through the dedicated buffer or through the weight ring."""
    cabi.set_tuning("ts.split", split)
    cabi.set_tuning("ts.slow_reduce", slow)
    w, s, z = synth.quantized_weight(384, 4096, 4, 64, seed=21)
    x = synth.activations((B, 4096), 22)
    want = oq.reference_q4_matvec_decode(x, w, s, z, group_size=64)
    d = lambda t: t.to(tcgen05)
    got = quant_ops.q4_matvec_decode(d(x), d(w), d(s), d(z), group_size=64)
    assert rel_l2(got, want) <= TOL


@pytest.mark.parametrize("bits", [4, 8])
def test_symmetric_codes_without_zero_points(tcgen05, bits):
    w, s, _ = synth.quantized_weight(512, 1024, bits, 64, seed=31)
    x = synth.activations((6, 1024), 32)
    want = _ref(bits)(x, w, s, None, group_size=64)
    got = _fn(bits)(x.to(tcgen05), w.to(tcgen05), s.to(tcgen05), None, group_size=64)
    assert rel_l2(got, want) <= TOL


def test_non_integer_and_negative_zero_points_and_scales(tcgen05):
    """The reference's own tests draw scales and zero points from N(0,1): any sign, any fraction."""
    g = torch.Generator().manual_seed(5)
    codes = torch.randint(0, 256, (256, 512), generator=g, dtype=torch.int32).to(torch.uint8)
    scales = torch.randn((256, 16), generator=g).to(torch.float16)
    zeros = (torch.randn((256, 16), generator=g) * 3 + 7.3).to(torch.float16)
    x = synth.activations((9, 1024), 6)
    want = oq.reference_q4_matvec_decode(x, codes, scales, zeros, group_size=64)
    d = lambda t: t.to(tcgen05)
    got = quant_ops.q4_matvec_decode(d(x), d(codes), d(scales), d(zeros), group_size=64)
    assert rel_l2(got, want) <= TOL


@pytest.mark.parametrize("bits,B,N,K", [(4, 1, 512, 1024), (4, 8, 14336, 4096), (4, 32, 1792, 4096), (8, 3, 1024, 1024)])
@pytest.mark.parametrize("big", [-1, 1])
def test_gate_up_swiglu(tcgen05, bits, B, N, K, big):
    cabi.set_tuning("ts.big", big)
    gw, gs, gz = synth.quantized_weight(N, K, bits, 64, seed=41)
    uw, us, uz = synth.quantized_weight(N, K, bits, 64, seed=42)
    x = synth.activations((B, K), 43)
    wg = _ref(bits)(x, gw, gs, gz, group_size=64)
    wu = _ref(bits)(x, uw, us, uz, group_size=64)
    d = lambda t: t.to(tcgen05)
    out = quant_ops.gate_up_rows(bits, d(x), d(gw), d(uw), d(gs), d(us), d(gz), d(uz), 64, want_gate_up=True, want_act=True)
    gate, up, act = out["gate"], out["up"], out["act"]
    assert rel_l2(gate, wg) <= TOL and rel_l2(up, wu) <= TOL
    # SwiGLU is applied to the kernel's own (rounded) gate / up rows
    assert rel_l2(act, reference_swiglu(gate.cpu(), up.cpu())) <= 2e-4


@pytest.mark.parametrize("B,with_res", [(1, False), (6, True), (32, True)])
@pytest.mark.parametrize("big", [-1, 1])
@pytest.mark.parametrize("fuse_norm", [1, 0])
def test_fused_norm_prologue_and_residual_epilogue(tcgen05, B, with_res, big, fuse_norm):
    """quantized_mlp_block through the tcgen05 kernel: [add + rmsnorm + gate/up + SwiGLU] and [down + residual], the
    norm in the kernel's prologue (fuse_norm) or as the row kernel's launch in front of it (the default)."""
    cabi.set_tuning("ts.big", big)
    cabi.set_tuning("gemv.fuse_norm", fuse_norm)
    hidden, inter = 1024, 2048
    gw, gs, gz = synth.quantized_weight(inter, hidden, 4, 64, seed=51)
    uw, us, uz = synth.quantized_weight(inter, hidden, 4, 64, seed=52)
    dw, ds, dz = synth.quantized_weight(hidden, inter, 4, 64, seed=53)
    x = synth.activations((B, 1, hidden), 54)
    res = synth.activations((B, 1, hidden), 55) if with_res else torch.zeros_like(x)
    nw = (torch.rand(hidden, generator=torch.Generator().manual_seed(56)) + 0.5).to(torch.float16)
    from oracle import mlp_block_ops as om
    want, wi = om.reference_quantized_mlp_block(x, res, nw, gw, gs, uw, us, dw, ds, gate_zeros=gz, up_zeros=uz,
                                                down_zeros=dz, bits=4, group_size=64, return_intermediates=True)
    d = lambda t: t.to(tcgen05)
    got, gi = mlp_ops.quantized_mlp_block(d(x), d(res), d(nw), d(gw), d(gs), d(uw), d(us), d(dw), d(ds), gate_zeros=d(gz),
                                          up_zeros=d(uz), down_zeros=d(dz), bits=4, group_size=64,
                                          backend_preset="fused_experimental", return_intermediates=True)
    assert torch.equal(gi["z"].cpu(), wi["z"])
    for key in ("normed", "gate", "up", "mlp", "down"):
        assert rel_l2(gi[key], wi[key]) <= TOL, key
    assert rel_l2(got, want) <= TOL


@pytest.mark.parametrize("bits,B,N,K,world", [(4, 8, 4096, 4096, 2), (4, 32, 4096, 14336, 4), (4, 16, 6144, 4096, 8),
                                              (8, 6, 2048, 2048, 2)])
def test_row_shards_reproduce_the_unsharded_rows_bit_for_bit(tcgen05, bits, B, N, K, world):
    """Tensor parallelism shards the weight rows.  With "ts.tp_world" set, a shard's launch splits K exactly as the
    unsharded launch does, so its rows are the unsharded rows bit for bit - on either shape of the kernel."""
    w, s, z = synth.quantized_weight(N, K, bits, 64, seed=71)
    x = synth.activations((B, K), 72)
    d = lambda t: t.to(tcgen05).contiguous()
    full = _fn(bits)(d(x), d(w), d(s), d(z), group_size=64)
    assert rel_l2(full, _ref(bits)(x, w, s, z, group_size=64)) <= TOL
    per = N // world
    try:
        for big in (-1, 1):
            cabi.set_tuning("ts.tp_world", world)
            cabi.set_tuning("ts.big", big)
            for r in (0, world - 1):
                rows = slice(r * per, (r + 1) * per)
                part = _fn(bits)(d(x), d(w[rows]), d(s[rows]), d(z[rows]), group_size=64)
                assert torch.equal(part, full[:, rows]), (big, r)
    finally:
        cabi.set_tuning("ts.tp_world", 0)


def test_default_routing_takes_batches_of_five_and_more(cuda):
    """With no tuning set, batch 4 runs the mma.sync kernel and batch 5 the tcgen05 kernel; both agree with the
    oracle, and with each other to within the parity bound."""
    for key in ("gemv.ts", "ts.big"):
        cabi.set_tuning(key, 0)
    w, s, z = synth.quantized_weight(1024, 2048, 4, 64, seed=61)
    x = synth.activations((5, 2048), 62)
    want = oq.reference_q4_matvec_decode(x, w, s, z, group_size=64)
    d = lambda t: t.to(cuda)
    y5 = quant_ops.q4_matvec_decode(d(x), d(w), d(s), d(z), group_size=64)
    y4 = quant_ops.q4_matvec_decode(d(x[:4]), d(w), d(s), d(z), group_size=64)
    assert rel_l2(y5, want) <= TOL and rel_l2(y4, want[:4]) <= TOL
    cabi.set_tuning("gemv.ts", -1)
    y5_old = quant_ops.q4_matvec_decode(d(x), d(w), d(s), d(z), group_size=64)
    cabi.set_tuning("gemv.ts", 0)
    assert rel_l2(y5, y5_old) <= TOL
    assert cabi.device_status() == 0
