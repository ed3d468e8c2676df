"""Loader for the reference's quantized checkpoint package: ``package.json`` + ``tensors/*.npy``.

Format (models/quantized_package_io.py:39-150, models/quantized_package_writer.py:51-190,
docs/quantized_package_tensor_data.md): ``package.json`` holds the model config, the quantisation
settings and, per layer, one metadata record per tensor key (``qkv``, ``o_proj``, ``gate_proj``,
``up_proj``, ``down_proj`` with ``data_file`` = packed codes and ``scales_file``, optionally
``zeros_file``; ``input_layernorm`` / ``post_attention_layernorm`` with ``data_file`` only, bits 0).
File names are relative to the tensor directory (``tensors/`` beside ``package.json``); ``checksum``
is the sha256 of the data file.  Symmetric packages carry no zeros: the kernels get a materialised
zero point of 8 (q4) or 128 (q8) per group, as models/quantized_layer_package.py:27-28 does.

The loader reads the files with numpy, checks shapes, dtypes and checksums against the metadata
and puts the tensors on a device, in the layout ``stack.DecodeStack`` and the operators take
(codes uint8 ``[N, K/2 | K]``, scales and zeros ``[N, K/G]`` fp16).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

import numpy as np
import torch

REQUIRED_LAYER_TENSOR_KEYS = ("input_layernorm", "post_attention_layernorm", "qkv", "o_proj", "gate_proj", "up_proj",
                              "down_proj")
LINEAR_KEYS = ("qkv", "o_proj", "gate_proj", "up_proj", "down_proj")
VALID_ROLES = ("qkv", "o_proj", "gate_proj", "up_proj", "down_proj", "embedding", "lm_head", "norm", "final_norm",
               "other")
FORMAT_VERSION = "0.1.0"


class PackageError(ValueError):
    """The package on disk does not match its own metadata (missing file, shape, dtype, checksum)."""


@dataclass
class QuantizedTensorMetadata:
    name: str
    role: str
    bits: int
    group_size: int
    original_shape: tuple[int, ...]
    packed_shape: tuple[int, ...]
    scales_shape: tuple[int, ...]
    zeros_shape: tuple[int, ...] | None = None
    dtype: str = "float16"
    data_file: str | None = None
    scales_file: str | None = None
    zeros_file: str | None = None
    checksum: str | None = None

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "QuantizedTensorMetadata":
        zeros_shape = data.get("zeros_shape")
        return cls(name=data["name"], role=data["role"], bits=int(data["bits"]), group_size=int(data["group_size"]),
                   original_shape=tuple(data["original_shape"]), packed_shape=tuple(data["packed_shape"]),
                   scales_shape=tuple(data["scales_shape"]),
                   zeros_shape=None if zeros_shape is None else tuple(zeros_shape), dtype=data.get("dtype", "float16"),
                   data_file=data.get("data_file"), scales_file=data.get("scales_file"),
                   zeros_file=data.get("zeros_file"), checksum=data.get("checksum"))


@dataclass
class QuantizedLayerMetadata:
    layer_idx: int
    tensors: dict[str, QuantizedTensorMetadata]

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "QuantizedLayerMetadata":
        return cls(layer_idx=int(data["layer_idx"]),
                   tensors={k: QuantizedTensorMetadata.from_dict(v) for k, v in data.get("tensors", {}).items()})


@dataclass
class QuantizedCheckpointPackage:
    format_version: str = FORMAT_VERSION
    model_type: str = "llama_like"
    config: dict[str, Any] = field(default_factory=dict)
    quantization: dict[str, Any] = field(default_factory=dict)
    layers: list[QuantizedLayerMetadata] = field(default_factory=list)
    global_tensors: dict[str, QuantizedTensorMetadata] = field(default_factory=dict)
    metadata: dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "QuantizedCheckpointPackage":
        return cls(format_version=data.get("format_version", FORMAT_VERSION), model_type=data.get("model_type", "llama_like"),
                   config=data.get("config", {}), quantization=data.get("quantization", {}),
                   layers=[QuantizedLayerMetadata.from_dict(d) for d in data.get("layers", [])],
                   global_tensors={k: QuantizedTensorMetadata.from_dict(v) for k, v in data.get("global_tensors", {}).items()},
                   metadata=data.get("metadata", {}))

    @classmethod
    def load_json(cls, path) -> "QuantizedCheckpointPackage":
        return cls.from_dict(json.loads(Path(path).read_text(encoding="utf-8")))

    def validate(self) -> "QuantizedCheckpointPackage":
        """The structural rules of models/quantized_package_io.py:214-279 for a complete package."""
        if not self.format_version:
            raise ValueError("format_version must be non-empty")
        if not self.model_type:
            raise ValueError("model_type must be non-empty")
        if not self.layers:
            raise ValueError("package must contain at least one layer unless allow_partial=True")
        seen: set[int] = set()
        for layer in self.layers:
            if layer.layer_idx < 0:
                raise ValueError(f"layer_idx must be non-negative, got {layer.layer_idx}")
            if layer.layer_idx in seen:
                raise ValueError(f"duplicate layer_idx: {layer.layer_idx}")
            seen.add(layer.layer_idx)
            for key in REQUIRED_LAYER_TENSOR_KEYS:
                if key not in layer.tensors:
                    raise ValueError(f"layer {layer.layer_idx} missing required tensor key: {key!r}")
            for tensor in layer.tensors.values():
                if any(dim <= 0 for dim in tensor.original_shape):
                    raise ValueError(f"tensor {tensor.name!r} original_shape contains non-positive dims: {tensor.original_shape}")
                if tensor.role not in VALID_ROLES:
                    raise ValueError(f"tensor {tensor.name!r} has invalid role {tensor.role!r}; expected one of {list(VALID_ROLES)}")
                if tensor.role in ("norm", "final_norm"):
                    if tensor.bits != 0:
                        raise ValueError(f"tensor {tensor.name!r} is unquantized norm metadata and must use bits=0, got {tensor.bits}")
                    if tensor.group_size != 0:
                        raise ValueError(f"tensor {tensor.name!r} is unquantized norm metadata and must use group_size=0, got {tensor.group_size}")
                    continue
                if tensor.bits not in (4, 8):
                    raise ValueError(f"tensor {tensor.name!r} bits must be 4 or 8, got {tensor.bits}")
                if tensor.group_size <= 0:
                    raise ValueError(f"tensor {tensor.name!r} group_size must be positive, got {tensor.group_size}")
        lo, hi = min(seen), max(seen)
        if seen != set(range(lo, hi + 1)):
            raise ValueError(f"layer indices must be contiguous from {lo} to {hi}, missing indices: "
                             f"{sorted(set(range(lo, hi + 1)) - seen)}")
        return self


def compute_file_checksum(file_path, algorithm: str = "sha256") -> str:
    h = hashlib.new(algorithm)
    with Path(file_path).open("rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def load_tensor_npy(file_path) -> np.ndarray:
    """One ``.npy`` payload (models/tensor_data_io.py:47-50); pickled arrays are refused."""
    with Path(file_path).open("rb") as f:
        return np.load(f, allow_pickle=False)


def symmetric_zero_point(bits: int) -> float:
    if bits == 4:
        return 8.0
    if bits == 8:
        return 128.0
    raise ValueError(f"bits must be 4 or 8, got {bits}")


@dataclass
class LoadedPackage:
    package: QuantizedCheckpointPackage
    layers: list[dict]                    # per layer: input_norm, post_norm, qkv/o/gate/up/down = (codes, scales, zeros)
    global_tensors: dict[str, torch.Tensor]
    bits: int
    group_size: int
    bytes_loaded: int

    def stack_config(self, **overrides):
        """A ``stack.StackConfig`` with the dimensions of the package's model config."""
        from .stack import StackConfig
        c = self.package.config
        fields = dict(hidden=c["hidden_size"], intermediate=c["intermediate_size"], n_layers=len(self.layers),
                      n_heads=c["num_attention_heads"], n_kv_heads=c["num_key_value_heads"], head_dim=c["head_dim"],
                      rope_theta=float(c.get("rope_theta", 10000.0)), eps=float(c.get("rms_norm_eps", 1e-5)),
                      vocab=int(c.get("vocab_size") or 0), bits=self.bits, group_size=self.group_size)
        fields.update(overrides)
        return StackConfig(**fields)


def _resolve(package_dir: Path, tensor_subdir: str, rel: str) -> Path:
    p = Path(rel)
    if p.is_absolute():
        return p
    for base in (package_dir / tensor_subdir, package_dir):
        if (base / p).exists():
            return base / p
    raise PackageError(f"tensor file not found: {rel} (looked in {package_dir / tensor_subdir} and {package_dir})")


def _to_float_tensor(arr: np.ndarray, what: str, device, dtype) -> torch.Tensor:
    if arr.dtype.kind != "f":
        raise PackageError(f"{what}: expected a floating-point array, got {arr.dtype}")
    return torch.from_numpy(np.ascontiguousarray(arr)).to(device=device, dtype=dtype)


def load_quantized_package(package_dir, device="cuda", *, tensor_subdir: str = "tensors", check_checksums: bool = True,
                           scale_dtype: torch.dtype = torch.float16, norm_dtype: torch.dtype = torch.float16) -> LoadedPackage:
    """Reads ``package_dir/package.json`` and every tensor file it names; returns device tensors.

    Checks, per linear: codes are uint8 of ``packed_shape`` = ``[N, ceil(K/2)]`` (q4) or ``[N, K]`` (q8) for
    ``original_shape`` ``[N, K]``; scales (and zeros, when a file is given) are ``[N, ceil(K/group_size)]``; the
    data file's sha256 equals ``checksum``.  Missing zeros become the symmetric zero point."""
    package_dir = Path(package_dir)
    package = QuantizedCheckpointPackage.load_json(package_dir / "package.json").validate()
    total = 0

    def read(rel, what, checksum=None):
        nonlocal total
        if rel is None:
            raise PackageError(f"{what}: no file recorded in package.json (metadata-only package)")
        path = _resolve(package_dir, tensor_subdir, rel)
        if check_checksums and checksum is not None:
            got = compute_file_checksum(path)
            if got != checksum:
                raise PackageError(f"{what}: checksum mismatch for {path.name}: expected {checksum}, got {got}")
        arr = load_tensor_npy(path)
        total += arr.nbytes
        return arr

    layers = []
    for layer in sorted(package.layers, key=lambda l: l.layer_idx):
        out: dict[str, Any] = {}
        for key, dst in (("input_layernorm", "input_norm"), ("post_attention_layernorm", "post_norm")):
            meta = layer.tensors[key]
            arr = read(meta.data_file, meta.name, meta.checksum)
            if tuple(arr.shape) != tuple(meta.original_shape):
                raise PackageError(f"{meta.name}: shape {tuple(arr.shape)} != original_shape {tuple(meta.original_shape)}")
            out[dst] = _to_float_tensor(arr, meta.name, device, norm_dtype)
        for key, dst in zip(LINEAR_KEYS, ("qkv", "o", "gate", "up", "down")):
            meta = layer.tensors[key]
            if len(meta.original_shape) != 2:
                raise PackageError(f"{meta.name}: original_shape must be [N, K], got {tuple(meta.original_shape)}")
            N, K = meta.original_shape
            want_codes = (N, (K + 1) // 2 if meta.bits == 4 else K)
            want_groups = (N, (K + meta.group_size - 1) // meta.group_size)
            codes = read(meta.data_file, meta.name, meta.checksum)
            if codes.dtype != np.uint8:
                raise PackageError(f"{meta.name}: packed codes must be uint8, got {codes.dtype}")
            if tuple(codes.shape) != want_codes or tuple(meta.packed_shape) != want_codes:
                raise PackageError(f"{meta.name}: packed codes {tuple(codes.shape)} (metadata {tuple(meta.packed_shape)}) "
                                   f"!= {want_codes} for a q{meta.bits} [{N}, {K}] weight")
            scales = read(meta.scales_file, f"{meta.name}.scales")
            if tuple(scales.shape) != want_groups:
                raise PackageError(f"{meta.name}: scales {tuple(scales.shape)} != {want_groups}")
            scales_t = _to_float_tensor(scales, f"{meta.name}.scales", device, scale_dtype)
            if meta.zeros_file is not None:
                zeros = read(meta.zeros_file, f"{meta.name}.zeros")
                if tuple(zeros.shape) != want_groups:
                    raise PackageError(f"{meta.name}: zeros {tuple(zeros.shape)} != {want_groups}")
                zeros_t = _to_float_tensor(zeros, f"{meta.name}.zeros", device, scale_dtype)
            else:
                zeros_t = torch.full_like(scales_t, symmetric_zero_point(meta.bits))
            out[dst] = (torch.from_numpy(np.ascontiguousarray(codes)).to(device), scales_t, zeros_t)
        layers.append(out)

    linear_meta = [layer.tensors[k] for layer in package.layers for k in LINEAR_KEYS]
    bits = {m.bits for m in linear_meta}
    groups = {m.group_size for m in linear_meta}
    if len(bits) != 1 or len(groups) != 1:
        raise PackageError(f"mixed quantisation inside one package is not supported: bits {sorted(bits)}, group sizes {sorted(groups)}")

    global_tensors = {}
    for name, meta in package.global_tensors.items():
        if meta.data_file is None:
            continue
        arr = read(meta.data_file, f"global_tensors.{name}", meta.checksum)
        if tuple(arr.shape) != tuple(meta.original_shape):
            raise PackageError(f"global_tensors.{name}: shape {tuple(arr.shape)} != original_shape {tuple(meta.original_shape)}")
        global_tensors[name] = _to_float_tensor(arr, f"global_tensors.{name}", device, norm_dtype)
    return LoadedPackage(package=package, layers=layers, global_tensors=global_tensors, bits=bits.pop(),
                         group_size=groups.pop(), bytes_loaded=total)
