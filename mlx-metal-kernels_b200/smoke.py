"""One small invocation of every hot-path kernel on cuda:0, checked against the CPU oracle.

Run through ``__graft_entry__.smoke()``.  The oracle (``oracle/`` at the repository root) is
imported here only as the checker.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

from . import synth
from .ops import _cabi, mlp_block_ops, paged_quantized_kv_ops as pq, quant_ops


def _rel(a, b):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    return float((a - b).norm() / b.norm())


def run() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("smoke() needs a CUDA device: the library has no CPU route")
    root = Path(__file__).resolve().parents[1]
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    from oracle import mlp_block_ops as om, paged_quantized_kv_ops as opq, quant_ops as oq

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    _cabi.load()
    d = lambda t: None if t is None else t.to(dev)

    # q4 matvec, tensor-core path
    w, s, z = synth.quantized_weight(512, 1024, 4, 64, seed=1)
    x = synth.activations((1, 1024), 2)
    y = quant_ops.q4_matvec_decode(d(x), d(w), d(s), d(z), group_size=64, backend="cuda")
    err = _rel(y, oq.reference_q4_matvec_decode(x, w, s, z, group_size=64))
    assert err <= 1e-3, f"q4 matvec rel-L2 {err}"
    # q4 / q8 matvec at batch 8: the tcgen05 kernel (TMA-tiled codes, weights dequantised into tensor memory)
    for bits in (4, 8):
        w8, s8, z8 = synth.quantized_weight(384, 1024, bits, 64, seed=11 + bits)
        x8 = synth.activations((8, 1024), 12)
        fn = quant_ops.q4_matvec_decode if bits == 4 else quant_ops.q8_matvec_decode
        ref = oq.reference_q4_matvec_decode if bits == 4 else oq.reference_q8_matvec_decode
        err = _rel(fn(d(x8), d(w8), d(s8), d(z8), group_size=64, backend="cuda"), ref(x8, w8, s8, z8, group_size=64))
        assert err <= 1e-3, f"q{bits} batch-8 matvec rel-L2 {err}"
    # bit-exact dequant
    deq = quant_ops.dequant_q4(d(w), d(s), d(z), group_size=64)
    assert torch.equal(deq.cpu(), oq.reference_dequant_q4(w, s, z, group_size=64)), "dequant not bit-exact"

    # fused MLP block
    gw, gs, gz = synth.quantized_weight(1024, 512, 4, 64, seed=3)
    uw, us, uz = synth.quantized_weight(1024, 512, 4, 64, seed=4)
    dw, ds, dz = synth.quantized_weight(512, 1024, 4, 64, seed=5)
    h = synth.activations((2, 1, 512), 6)
    nw = torch.ones(512, dtype=torch.float16)
    out = mlp_block_ops.quantized_mlp_block(d(h), d(torch.zeros_like(h)), d(nw), d(gw), d(gs), d(uw), d(us), d(dw), d(ds),
                                            gate_zeros=d(gz), up_zeros=d(uz), down_zeros=d(dz), bits=4, group_size=64,
                                            backend_preset="cuda")
    want = om.reference_quantized_mlp_block(h, torch.zeros_like(h), nw, gw, gs, uw, us, dw, ds, gate_zeros=gz,
                                            up_zeros=uz, down_zeros=dz, bits=4, group_size=64)
    err = _rel(out, want)
    assert err <= 1e-3, f"mlp block rel-L2 {err}"

    # paged q4 / q8 GQA decode attention, ragged lengths: batch 3 runs the one-launch cluster kernel, batch 6 the
    # split-KV kernel with its merge
    for bits, B in ((4, 3), (8, 6)):
        case = synth.paged_kv_case(B, 8, 128, 16, num_pages=40 * B, min_len=5, max_len=300, bits=bits, group_size=32, seed=7)
        q = synth.activations((B, 1, 32, 128), 8)
        cache = pq.PagedQuantizedKVCache(**{k: (d(v) if torch.is_tensor(v) else v) for k, v in case.items()})
        o = pq.paged_quantized_kv_gqa_decode_attention(d(q), cache, backend="cuda")
        ocache = opq.OraclePagedKV(**case)
        want = opq.reference_paged_quantized_kv_gqa_decode_attention(q, ocache)
        err = float((o.cpu().float() - want.float()).abs().max())
        assert err <= 2e-3, f"q{bits} paged attention max abs err {err}"
    torch.cuda.synchronize()
    status = _cabi.device_status()
    assert status == 0, f"device status word {status}"
    print("smoke ok")
