"""Shared builders for the parity tests: seeded inputs on CPU, moved to the GPU by the caller."""
from __future__ import annotations

import importlib

import torch

import __graft_entry__ as entry

entry.load_package()
synth = importlib.import_module("mlx_metal_kernels_b200.synth")
cabi = importlib.import_module("mlx_metal_kernels_b200.ops._cabi")
quant_ops = importlib.import_module("mlx_metal_kernels_b200.ops.quant_ops")
mlp_ops = importlib.import_module("mlx_metal_kernels_b200.ops.mlp_block_ops")
pq_ops = importlib.import_module("mlx_metal_kernels_b200.ops.paged_quantized_kv_ops")
qkv_ops = importlib.import_module("mlx_metal_kernels_b200.ops.quantized_kv_cache_ops")
pkv_ops = importlib.import_module("mlx_metal_kernels_b200.ops.paged_kv_ops")
sparse_ops = importlib.import_module("mlx_metal_kernels_b200.ops.sparse_attention_ops")
act_ops = importlib.import_module("mlx_metal_kernels_b200.ops.activation_ops")
norm_ops = importlib.import_module("mlx_metal_kernels_b200.ops.norm_ops")
fused_ops = importlib.import_module("mlx_metal_kernels_b200.ops.fused_ops")


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def random_quant_case(bits, N, K, G, seed, *, zeros="float", scale_dtype=torch.float32, scale_kind="normal"):
    """Random codes / scales / zeros in the style of the reference's unit tests: scales ~N(0,1)
    (negative values occur) or U(0.01, 0.1); zeros None, or float and non-integer."""
    g = gen(seed)
    cols = (K + 1) // 2 if bits == 4 else K
    codes = torch.randint(0, 256, (N, cols), generator=g, dtype=torch.int32).to(torch.uint8)
    groups = (K + G - 1) // G
    if scale_kind == "normal":
        scales = torch.randn((N, groups), generator=g)
    else:
        scales = torch.rand((N, groups), generator=g) * 0.09 + 0.01
    z = None
    if zeros == "float":
        z = torch.randn((N, groups), generator=g) * (2.0 if bits == 4 else 16.0) + (8.0 if bits == 4 else 128.0)
        z = z.to(scale_dtype)
    return codes, scales.to(scale_dtype), z


def to_dev(device, *tensors):
    return [None if t is None else t.to(device) for t in tensors]


def rel_l2(a, b):
    a = a.detach().to("cpu", torch.float64)
    b = b.detach().to("cpu", torch.float64)
    denom = float(b.norm())
    return float((a - b).norm()) / (denom if denom > 0 else 1.0)
