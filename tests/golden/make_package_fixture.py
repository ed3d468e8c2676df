"""Writes tests/golden/tiny_q4_package/ with the reference's own quantiser and package writer.

Run in a container that has the reference checkout (first argument, or $MLX_METAL_KERNELS_REF):

    python tests/golden/make_package_fixture.py [/path/to/reference]

The reference modules used (``models/quantize_weights.py``, ``models/quantized_layer_package.py``,
``models/quantized_package_io.py``, ``models/quantized_package_writer.py``) need numpy only.  The
package is a two-layer llama-like model small enough to commit (hidden 128, one head of dim 128,
q4 group 32, symmetric: no zeros files), plus ``expected_dequant.npz`` with the reference's own fp32
dequantisation of every 8th row of every linear rounded to fp16 (round to nearest even, the cast the MLX path
applies), which the loader test compares against.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
DEST = HERE / "tiny_q4_package"
ROLES = ("qkv", "o_proj", "gate_proj", "up_proj", "down_proj")


def main():
    ref_root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["MLX_METAL_KERNELS_REF"])
    sys.path.insert(0, str(ref_root))
    from models.llama_config import LlamaLikeConfig
    from models.quantize_weights import QuantizationConfig, dequantize_quantized_weight, quantize_weight_groupwise
    from models.quantized_layer_package import QuantizedLinearPackage, QuantizedLlamaLayerPackage
    from models.quantized_package_io import QuantizedTensorMetadata, package_from_quantized_layers
    from models.quantized_package_writer import PackageWriterConfig, QuantizedPackageWriter

    cfg = LlamaLikeConfig(hidden_size=128, intermediate_size=256, num_attention_heads=1, num_key_value_heads=1,
                          head_dim=128, num_hidden_layers=2, max_position_embeddings=64, rope_theta=10000.0,
                          rms_norm_eps=1e-5, vocab_size=32, model_type="llama_like_tiny_fixture").validate()
    bits, G = 4, 32
    qcfg = QuantizationConfig(bits=bits, group_size=G)
    rng = np.random.default_rng(424242)
    shapes = {"qkv": (3 * 128, 128), "o_proj": (128, 128), "gate_proj": (256, 128), "up_proj": (256, 128),
              "down_proj": (128, 256)}
    layers, expected = [], {}
    for idx in range(cfg.num_hidden_layers):
        linears = {}
        for role in ROLES:
            w = (rng.standard_normal(shapes[role]) * 0.05).astype(np.float32)
            qw = quantize_weight_groupwise(w, qcfg)
            linears[role] = QuantizedLinearPackage(name=f"layers.{idx}.{role}", weight=qw.packed_weight, scales=qw.scales,
                                                   zeros=None, bits=bits, group_size=G, original_shape=shapes[role])
            expected[f"layers.{idx}.{role}"] = np.asarray(
                dequantize_quantized_weight(qw.packed_weight, qw.scales, None, bits=bits, group_size=G), dtype=np.float32
            ).astype(np.float16)[::8]
        layers.append(QuantizedLlamaLayerPackage(
            layer_idx=idx,
            input_layernorm_weight=(rng.random(128) + 0.5).astype(np.float16),
            post_attention_layernorm_weight=(rng.random(128) + 0.5).astype(np.float16),
            qkv=linears["qkv"], o_proj=linears["o_proj"], gate_proj=linears["gate_proj"], up_proj=linears["up_proj"],
            down_proj=linears["down_proj"]))
    package = package_from_quantized_layers(cfg, layers, bits=bits, group_size=G, metadata={"source": "synthetic fixture"})
    embedding = rng.standard_normal((cfg.vocab_size, 128)).astype(np.float16)
    final_norm = (rng.random(128) + 0.5).astype(np.float16)
    for name, role, arr in (("embedding", "embedding", embedding), ("norm", "final_norm", final_norm)):
        package.global_tensors[name] = QuantizedTensorMetadata(
            name=name, role=role, bits=0, group_size=0, original_shape=tuple(arr.shape), packed_shape=tuple(arr.shape),
            scales_shape=(0,), dtype="float16")
    if DEST.exists():
        shutil.rmtree(DEST)
    report = QuantizedPackageWriter(PackageWriterConfig(tensor_subdir="tensors")).write_tensors(
        package, layers, DEST, global_tensors={"embedding": embedding, "norm": final_norm})
    if not report.ok:
        raise SystemExit(f"writer reported errors: {report.errors}")
    np.savez_compressed(DEST / "expected_dequant.npz", **expected)
    total = sum(f.stat().st_size for f in DEST.rglob("*") if f.is_file())
    print(f"wrote {DEST} ({report.tensor_count} tensors, {total} bytes on disk)")


if __name__ == "__main__":
    main()
