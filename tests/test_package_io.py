"""Loader of the reference's quantized checkpoint package (package.json + tensors/*.npy) against a
package written by the reference's own writer (tests/golden/tiny_q4_package, made by
tests/golden/make_package_fixture.py)."""
import importlib
import json
import shutil
from pathlib import Path

import numpy as np
import pytest
import torch

import __graft_entry__ as entry
from helpers import cabi, quant_ops, rel_l2
from oracle import paged_quantized_kv_ops as opq, quant_ops as oq, stack as ostack

entry.load_package()
package_io = importlib.import_module("mlx_metal_kernels_b200.package_io")
stack_mod = importlib.import_module("mlx_metal_kernels_b200.stack")
FIXTURE = Path(__file__).resolve().parent / "golden" / "tiny_q4_package"
NAMES = {"qkv": "qkv", "o": "o_proj", "gate": "gate_proj", "up": "up_proj", "down": "down_proj"}


def test_loads_the_reference_writers_package_on_cpu_tensors():
    loaded = package_io.load_quantized_package(FIXTURE, "cpu")
    assert loaded.bits == 4 and loaded.group_size == 32 and len(loaded.layers) == 2
    assert loaded.package.config["hidden_size"] == 128 and loaded.package.quantization["symmetric"] is True
    expected = np.load(FIXTURE / "expected_dequant.npz")
    shapes = {"qkv": (384, 128), "o": (128, 128), "gate": (256, 128), "up": (256, 128), "down": (128, 256)}
    for idx, layer in enumerate(loaded.layers):
        assert layer["input_norm"].shape == (128,) and layer["post_norm"].dtype == torch.float16
        for key, (N, K) in shapes.items():
            codes, scales, zeros = layer[key]
            assert codes.dtype == torch.uint8 and tuple(codes.shape) == (N, K // 2)
            assert scales.dtype == torch.float16 and tuple(scales.shape) == (N, K // 32)
            assert bool((zeros == 8.0).all()) and zeros.shape == scales.shape     # symmetric package: materialised zero point
            # the oracle's dequantisation of what was loaded equals the reference's own (every 8th row is stored)
            got = oq.reference_dequant_q4(codes, scales, zeros, group_size=32, out_dtype=torch.float16)
            want = torch.from_numpy(expected[f"layers.{idx}.{NAMES[key]}"])
            assert torch.equal(got[::8], want), (idx, key)
    assert set(loaded.global_tensors) == {"embedding", "norm"} and loaded.global_tensors["embedding"].shape == (32, 128)
    files = list((FIXTURE / "tensors").glob("*.npy"))
    assert loaded.bytes_loaded == sum(np.load(f).nbytes for f in files)
    cfg = loaded.stack_config(kv_bits=8)
    assert (cfg.hidden, cfg.intermediate, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.vocab, cfg.bits,
            cfg.group_size, cfg.rope_theta) == (128, 256, 2, 1, 1, 128, 32, 4, 32, 10000.0)


def test_loader_rejects_packages_that_do_not_match_their_metadata(tmp_path):
    def copy(name):
        dst = tmp_path / name
        shutil.copytree(FIXTURE, dst)
        return dst

    # a flipped byte in a data file: checksum mismatch (and accepted when checksums are switched off)
    pkg = copy("flipped")
    victim = pkg / "tensors" / "layers.1.o_proj.weight.npy"
    raw = bytearray(victim.read_bytes())
    raw[-1] ^= 0x10
    victim.write_bytes(bytes(raw))
    with pytest.raises(package_io.PackageError, match="checksum mismatch"):
        package_io.load_quantized_package(pkg, "cpu")
    package_io.load_quantized_package(pkg, "cpu", check_checksums=False)

    pkg = copy("missing")
    (pkg / "tensors" / "layers.0.qkv.scales.npy").unlink()
    with pytest.raises(package_io.PackageError, match="tensor file not found"):
        package_io.load_quantized_package(pkg, "cpu")

    def edited(name, fn):
        pkg = copy(name)
        meta = json.loads((pkg / "package.json").read_text())
        fn(meta)
        (pkg / "package.json").write_text(json.dumps(meta))
        return pkg

    with pytest.raises(package_io.PackageError, match="packed codes"):
        package_io.load_quantized_package(edited("shape", lambda m: m["layers"][0]["tensors"]["qkv"].update(original_shape=[384, 256])), "cpu")
    with pytest.raises(ValueError, match="missing required tensor key"):
        package_io.load_quantized_package(edited("nokey", lambda m: m["layers"][1]["tensors"].pop("up_proj")), "cpu")
    with pytest.raises(ValueError, match="bits must be 4 or 8"):
        package_io.load_quantized_package(edited("bits", lambda m: m["layers"][0]["tensors"]["down_proj"].update(bits=3)), "cpu")
    with pytest.raises(ValueError, match="duplicate layer_idx"):
        package_io.load_quantized_package(edited("dup", lambda m: m["layers"][1].update(layer_idx=0)), "cpu")
    with pytest.raises(package_io.PackageError, match="metadata-only"):
        package_io.load_quantized_package(edited("nodata", lambda m: m["layers"][0]["tensors"]["gate_proj"].update(data_file=None)), "cpu")
    # explicit zeros files are honoured
    pkg = copy("zeros")
    np.save(pkg / "tensors" / "layers.0.qkv.zeros.npy", np.full((384, 4), 7.5, dtype=np.float16))
    meta = json.loads((pkg / "package.json").read_text())
    meta["layers"][0]["tensors"]["qkv"].update(zeros_file="layers.0.qkv.zeros.npy", zeros_shape=[384, 4])
    (pkg / "package.json").write_text(json.dumps(meta))
    loaded = package_io.load_quantized_package(pkg, "cpu")
    assert bool((loaded.layers[0]["qkv"][2] == 7.5).all()) and bool((loaded.layers[1]["qkv"][2] == 8.0).all())


@pytest.mark.gpu
def test_loaded_package_dequantises_bit_exact_and_runs_the_decode_stack(cuda):
    loaded = package_io.load_quantized_package(FIXTURE, cuda)
    expected = np.load(FIXTURE / "expected_dequant.npz")
    for idx, layer in enumerate(loaded.layers):
        for key, name in NAMES.items():
            codes, scales, zeros = layer[key]
            got = quant_ops.dequant_q4(codes, scales, zeros, group_size=32, backend="cuda")
            assert torch.equal(got.cpu()[::8], torch.from_numpy(expected[f"layers.{idx}.{name}"])), (idx, key)
    # one decode step of the loaded model against the CPU oracle on the same tensors
    cfg = loaded.stack_config(kv_bits=8, kv_group_size=32)
    batch, positions = 2, torch.tensor([20, 3], dtype=torch.int32)
    emb, final_norm = loaded.global_tensors["embedding"], loaded.global_tensors["norm"]
    stack = stack_mod.DecodeStack(cfg, loaded.layers, final_norm, emb, batch, 64, cuda)
    stack.set_context(0, seed=7)
    stack.positions.copy_(positions.to(cuda))
    stack.lengths.copy_((positions + 1).to(cuda))
    ocaches = [opq.OraclePagedKV(
        k_pages_q=c.k_codes.cpu().clone(), v_pages_q=c.v_codes.cpu().clone(), k_scales=c.k_scales.cpu().clone(),
        v_scales=c.v_scales.cpu().clone(), block_table=stack.block_table.cpu(), lengths=(positions + 1), bits=8,
        page_size=cfg.page_size, group_size=cfg.kv_group_size,
        original_page_shape=(stack.num_pages, cfg.page_size, cfg.n_kv_heads, cfg.head_dim)) for c in stack.caches]
    cpu_layers = [{k: (v.cpu() if torch.is_tensor(v) else tuple(t.cpu() for t in v)) for k, v in l.items()} for l in loaded.layers]
    tokens = torch.tensor([5, 31])
    cos, sin = ostack.rope_tables(cfg.head_dim, cfg.rope_theta, 64)
    want = ostack.stack_decode_step(tokens, emb.cpu(), cpu_layers, ocaches, final_norm.cpu(), cos, sin, positions,
                                    cfg.oracle_dict())
    got = stack.step(tokens.to(cuda))
    assert rel_l2(got, want.squeeze(1)) <= 3e-3          # two layers of 1e-3-class operators
    assert cabi.device_status() == 0
