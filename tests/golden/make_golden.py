"""Generates tests/golden/hotpath_golden.npz from code the reference itself ships.

Run in a container that has the reference checkout (first argument, or $MLX_METAL_KERNELS_REF) and
oracle/_ref/libmetalref.so built (``make -C oracle``):

    python tests/golden/make_golden.py [/path/to/reference]

Two sources, both the reference's own code, neither needing MLX:

* ``models/quantize_weights.py`` (numpy): symmetric group-wise quantiser, q4 packing and the fp32
  ``(q - zero) * scale`` dequantisation.
* the Metal kernel bodies under ``kernels/`` compiled as C++ (oracle/metal_shim.cpp): dequant,
  serial matvec, paged q4/q8 GQA decode attention (ragged lengths, permuted block table with -1
  entries), fused SwiGLU, block-table lookup, residual add, SwiGLU, and - on the shim's threadgroup emulator -
  RMSNorm, fused residual + RMSNorm, the ``parallel`` and ``tiled`` matvec bodies and the tiled gate/up body.

Inputs come from numpy's seeded generator and are stored next to the outputs, so the fixtures
are self-contained.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import metal_ref  # noqa: E402


def _load_reference_quantizer(ref_root: Path):
    spec = importlib.util.spec_from_file_location("ref_quantize_weights", ref_root / "models" / "quantize_weights.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    ref_root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["MLX_METAL_KERNELS_REF"])
    qw = _load_reference_quantizer(ref_root)
    rng = np.random.default_rng(20240607)
    out = {}

    # --- numpy quantiser / packer / dequantiser of the reference -----------------------------
    for bits in (4, 8):
        for tag, (N, K, G) in {"a": (6, 96, 32), "b": (5, 80, 16)}.items():
            w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
            cfg = qw.QuantizationConfig(bits=bits, group_size=G, symmetric=True, dtype="float16")
            qt = qw.quantize_weight_groupwise(w, cfg)
            zeros = (rng.standard_normal(qt.scales.shape) * 4 + 8).astype(np.float32)
            key = f"np_q{bits}{tag}"
            out[f"{key}_w"] = w
            out[f"{key}_codes"] = np.asarray(qt.packed_weight)
            out[f"{key}_scales"] = np.asarray(qt.scales)
            out[f"{key}_G"] = np.int32(G)
            out[f"{key}_deq_sym"] = qw.dequantize_quantized_weight(qt.packed_weight, qt.scales, None, bits=bits, group_size=G)
            out[f"{key}_zeros"] = zeros
            out[f"{key}_deq_zero"] = qw.dequantize_quantized_weight(qt.packed_weight, qt.scales, zeros, bits=bits, group_size=G)
    codes = rng.integers(0, 16, size=(4, 63), dtype=np.uint8)
    out["np_pack_codes"] = codes
    out["np_pack_packed"] = qw._pack_q4_numpy(codes)

    # --- Metal kernel bodies run on the CPU ---------------------------------------------------
    for bits in (4, 8):
        M, K, G = 8, 128, 32
        cols = K // 2 if bits == 4 else K
        codes = rng.integers(0, 256, size=(M, cols), dtype=np.uint8)
        scales = rng.standard_normal((M, K // G)).astype(np.float16)
        zeros = (rng.standard_normal((M, K // G)) * 3 + (8 if bits == 4 else 128)).astype(np.float16)
        x = rng.standard_normal((2, K)).astype(np.float16)
        key = f"mtl_q{bits}"
        out[f"{key}_codes"], out[f"{key}_scales"], out[f"{key}_zeros"], out[f"{key}_x"] = codes, scales, zeros, x
        out[f"{key}_deq_zero"] = metal_ref.dequant(bits, codes, scales, zeros, G)
        out[f"{key}_deq_nozero"] = metal_ref.dequant(bits, codes, scales, None, G)
        out[f"{key}_matvec_zero"] = metal_ref.matvec(bits, x, codes, scales * np.float16(0.01), zeros, G)
        out[f"{key}_matvec_nozero"] = metal_ref.matvec(bits, x, codes, scales * np.float16(0.01), None, G)

    # paged attention: ragged lengths, shuffled pages, -1 beyond the length, G=32
    for bits in (4, 8):
        for tag, (B, Hq, Hkv, D, P, max_blocks, lengths) in {
            "gqa": (3, 8, 2, 64, 4, 6, [24, 7, 0]),
            "mqa": (2, 4, 1, 128, 16, 3, [33, 48]),
            "d16": (1, 4, 4, 16, 4, 4, [13]),
        }.items():
            num_pages = B * max_blocks + 3
            G = 32
            groups = (D + G - 1) // G
            cols = (D + 1) // 2 if bits == 4 else D
            kq = rng.integers(0, 256, size=(num_pages, P, Hkv, cols), dtype=np.uint8)
            vq = rng.integers(0, 256, size=(num_pages, P, Hkv, cols), dtype=np.uint8)
            smax = 7 if bits == 4 else 127
            ks = (np.abs(rng.standard_normal((num_pages, P, Hkv, groups))) * 2.5 / smax + 1e-3).astype(np.float16)
            vs = (np.abs(rng.standard_normal((num_pages, P, Hkv, groups))) * 2.5 / smax + 1e-3).astype(np.float16)
            perm = rng.permutation(num_pages).astype(np.int32)
            bt = np.full((B, max_blocks), -1, dtype=np.int32)
            cur = 0
            for b, L in enumerate(lengths):
                n = (L + P - 1) // P
                bt[b, :n] = perm[cur:cur + n]
                cur += n
            q = rng.standard_normal((B, 1, Hq, D)).astype(np.float16)
            scale = np.float32(1.0 / np.sqrt(D))
            o = metal_ref.paged_attention(bits, q, kq, vq, ks, vs, bt, np.asarray(lengths, np.int32),
                                          (num_pages, P, Hkv, D), G, float(scale))
            key = f"mtl_attn_q{bits}_{tag}"
            for name, val in dict(q=q, kq=kq, vq=vq, ks=ks, vs=vs, bt=bt, lengths=np.asarray(lengths, np.int32),
                                  shape=np.asarray((num_pages, P, Hkv, D), np.int32), out=o).items():
                out[f"{key}_{name}"] = val

    gate = (rng.standard_normal((3, 50)) * 3).astype(np.float16)
    up = rng.standard_normal((3, 50)).astype(np.float16)
    out["mtl_swiglu_gate"], out["mtl_swiglu_up"] = gate, up
    out["mtl_swiglu_out"] = metal_ref.fused_swiglu(gate, up)

    bt = rng.permutation(64).astype(np.int32).reshape(4, 16)
    pos = np.asarray([0, 17, 63, 126], dtype=np.int32)
    out["mtl_btl_table"], out["mtl_btl_pos"] = bt, pos
    out["mtl_btl_pages"], out["mtl_btl_offsets"] = metal_ref.block_table_lookup(bt, pos, 8)

    # contiguous quantised cache attention: ragged lengths, G=32; its own generator so that the arrays above
    # do not depend on what is added here
    rng2 = np.random.default_rng(20240607)
    for bits in (4, 8):
        for tag, (B, Hq, Hkv, D, max_s, lengths) in {
            "gqa": (3, 8, 2, 64, 24, [24, 7, 1]),
            "mqa": (2, 4, 1, 128, 48, [33, 48]),
            "d16": (1, 4, 4, 16, 13, [13]),
        }.items():
            G = 32
            groups = (D + G - 1) // G
            cols = (D + 1) // 2 if bits == 4 else D
            kq = rng2.integers(0, 256, size=(B, max_s, Hkv, cols), dtype=np.uint8)
            vq = rng2.integers(0, 256, size=(B, max_s, Hkv, cols), dtype=np.uint8)
            smax = 7 if bits == 4 else 127
            ks = (np.abs(rng2.standard_normal((B, max_s, Hkv, groups))) * 2.5 / smax + 1e-3).astype(np.float16)
            vs = (np.abs(rng2.standard_normal((B, max_s, Hkv, groups))) * 2.5 / smax + 1e-3).astype(np.float16)
            q = rng2.standard_normal((B, 1, Hq, D)).astype(np.float16)
            scale = np.float32(1.0 / np.sqrt(D))
            o = metal_ref.contiguous_attention(bits, q, kq, vq, ks, vs, np.asarray(lengths, np.int32),
                                               (B, max_s, Hkv, D), G, float(scale))
            key = f"mtl_cattn_q{bits}_{tag}"
            for name, val in dict(q=q, kq=kq, vq=vq, ks=ks, vs=vs, lengths=np.asarray(lengths, np.int32),
                                  shape=np.asarray((B, max_s, Hkv, D), np.int32), out=o).items():
                out[f"{key}_{name}"] = val

    # bodies that cooperate inside a threadgroup (run on the shim's threadgroup emulator), and the two element-wise
    # bodies added with them; a generator of their own keeps every array above unchanged
    rng3 = np.random.default_rng(20240608)
    x = rng3.standard_normal((2, 3, 200)).astype(np.float16)
    res = rng3.standard_normal((2, 3, 200)).astype(np.float16)
    w = (rng3.random(200) + 0.5).astype(np.float16)
    out["tg_norm_x"], out["tg_norm_res"], out["tg_norm_w"] = x, res, w
    out["tg_residual_add"] = metal_ref.residual_add(x, res)
    out["tg_swiglu"] = metal_ref.swiglu(x * np.float16(3), res)
    out["tg_rms_norm"] = metal_ref.rms_norm(x, w, 1e-5)
    out["tg_rmsnorm_residual_y"], out["tg_rmsnorm_residual_z"] = metal_ref.rmsnorm_residual(x, res, w, 1e-5)
    for bits in (4, 8):
        N, K, G = 10, 320, 32                       # N not a multiple of the 4-row tile
        cols = K // 2 if bits == 4 else K
        key = f"tg_q{bits}"
        codes = rng3.integers(0, 256, size=(N, cols), dtype=np.uint8)
        codes2 = rng3.integers(0, 256, size=(N, cols), dtype=np.uint8)
        scales = (rng3.standard_normal((N, K // G)) * 0.01).astype(np.float16)
        scales2 = (rng3.standard_normal((N, K // G)) * 0.01).astype(np.float16)
        zeros = (rng3.standard_normal((N, K // G)) * 3 + (8 if bits == 4 else 128)).astype(np.float16)
        xm = rng3.standard_normal((3, K)).astype(np.float16)
        for name, val in dict(codes=codes, codes2=codes2, scales=scales, scales2=scales2, zeros=zeros, x=xm).items():
            out[f"{key}_{name}"] = val
        out[f"{key}_parallel"] = metal_ref.matvec_parallel(bits, xm, codes, scales, zeros, G)
        out[f"{key}_tiled"] = metal_ref.matvec_tiled(bits, xm, codes, scales, zeros, G)
        out[f"{key}_tiled_nozero"] = metal_ref.matvec_tiled(bits, xm, codes, scales, None, G)
        out[f"{key}_gate"], out[f"{key}_up"] = metal_ref.gate_up_tiled(bits, xm, codes, codes2, scales, scales2, zeros, None, G)

    dest = Path(__file__).resolve().parent / "hotpath_golden.npz"
    np.savez_compressed(dest, **out)
    print(f"wrote {dest} ({dest.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    main()
