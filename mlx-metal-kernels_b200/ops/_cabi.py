"""ctypes binding of ``libb200q.so`` (C ABI declared in include/b200q.h).

Only device pointers, sizes and dtype codes cross this boundary; torch is used by the callers
for memory and streams.  There is no fallback: if the library is missing or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path

import torch

F16, BF16, F32 = 0, 1, 2
_PKG = Path(__file__).resolve().parents[1]
LIB_PATH = _PKG / "lib" / "libb200q.so"
HEADER_PATH = _PKG.parent / "include" / "b200q.h"

_c = ctypes
_vp, _i, _i64, _f, _sz = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_float, _c.c_size_t

# name -> (restype, argtypes); must list every function include/b200q.h declares
SIGNATURES = {
    "b200q_version": (_i, []),
    "b200q_strerror": (_c.c_char_p, [_i]),
    "b200q_device_status": (_i, [_i, _vp]),
    "b200q_set_tuning": (_i, [_c.c_char_p, _i]),
    "b200q_dequant": (_i, [_i, _vp, _vp, _vp, _vp, _i64, _i64, _i, _i, _i, _vp]),
    "b200q_qmatvec": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i, _i, _i, _vp]),
    "b200q_norm_qmatvec": (_i, [_i, _vp, _vp, _vp, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i, _i, _i,
                                _vp]),
    "b200q_rope_kv_append": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i64, _i, _i,
                                  _i, _vp]),
    "b200q_gate_up_swiglu": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _f, _vp, _vp,
                                  _i, _i64, _i64, _i, _i, _i, _vp]),
    "b200q_rope_append_paged_gqa_decode": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz,
                                                _i, _i, _i, _i, _i, _i64, _i, _i, _f, _vp]),
    "b200q_attention_stage_launches": (_i, [_i, _i, _i]),
    "b200q_quantize_kv": (_i, [_i, _vp, _vp, _vp, _i64, _i, _i, _i, _vp]),
    "b200q_peer_allgather": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _vp]),
    "b200q_tp_register": (_i, [_i, _vp, _vp, _vp, _vp, _i, _i]),
    "b200q_tp_next": (_i, [_i, _i]),
    "b200q_tp_set_packets": (_i, [_i, _i]),
    "b200q_wait_expiry_selftest": (_i, [_c.c_uint, _vp, _vp]),
    "b200q_swiglu": (_i, [_vp, _vp, _vp, _i64, _i64, _i, _vp]),
    "b200q_residual_add": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "b200q_rmsnorm_residual": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _f, _i, _i, _vp]),
    "b200q_block_table_lookup": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200q_paged_gqa_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "b200q_paged_gqa_static_scratch_bytes": (_sz, []),
    "b200q_paged_gqa_decode_static": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i64, _i, _i,
                                           _f, _i, _i, _vp]),
    "b200q_paged_gqa_decode": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i64,
                                    _i, _i, _f, _i, _i, _vp]),
    "b200q_paged_gqa_decode_window": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i64,
                                           _i, _i, _f, _i, _i, _i, _i, _vp]),
    "b200q_paged_gqa_decode_block_sparse": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _i, _i, _i,
                                                 _vp, _i, _i, _i, _i, _i, _i64, _i, _i, _f, _i, _i, _vp]),
    "b200q_paged_fp16_gqa_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "b200q_paged_fp16_gqa_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i64, _i, _f, _i,
                                         _vp]),
}

_lib = None


class B200QError(RuntimeError):
    """A libb200q call returned an error code."""


class ReferenceBackendUnavailable(RuntimeError):
    """``backend="reference"`` (or the CI safe-mode switch) was requested.

    The pure-MLX reference path belongs to the reference project; this library ships the CUDA
    backend only and has no CPU route."""


def header_functions() -> list[str]:
    """Names of the functions include/b200q.h declares."""
    text = HEADER_PATH.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", text)))


def load():
    """Loads the shared library and binds every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("B200Q_LIB", LIB_PATH))
    if not path.exists():
        raise B200QError(
            f"{path} not found: build it with `python {_PKG / 'build.py'}` (needs nvcc); "
            "there is no fallback implementation"
        )
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise B200QError(f"{path} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().b200q_strerror(rc).decode()
        raise B200QError(f"{what}: {msg} (code {rc})")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return F16
    if dtype == torch.bfloat16:
        return BF16
    if dtype == torch.float32:
        return F32
    raise TypeError(f"unsupported dtype {dtype}")


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise B200QError("the CUDA backend needs CUDA tensors; there is no CPU route in this library")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise B200QError(f"tensors live on different devices: {dev} and {t.device}")
    return dev


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def contiguous(t):
    return t if t is None or t.is_contiguous() else t.contiguous()


def scale_pair(scales, zeros):
    """Scales and zero points in one dtype the kernels read natively (fp16, bf16 or fp32).
    Differing or other dtypes are widened to fp32, which is exact."""
    ok = (torch.float16, torch.bfloat16, torch.float32)
    if scales.dtype in ok and (zeros is None or zeros.dtype == scales.dtype):
        return contiguous(scales), contiguous(zeros)
    return contiguous(scales.to(torch.float32)), (None if zeros is None else contiguous(zeros.to(torch.float32)))


def set_tuning(key: str, value: int) -> None:
    check(load().b200q_set_tuning(key.encode(), int(value)), "b200q_set_tuning")


def device_status(reset: bool = True) -> int:
    return load().b200q_device_status(int(reset), stream())


def safe_mode_enabled() -> bool:
    """The reference's CI switch that reroutes every Metal backend to the reference path
    (ops/quant_ops.py:33-34)."""
    return os.environ.get("MLX_METAL_CI_SAFE_MODE", "0") == "1"


def reference_unavailable(what: str):
    raise ReferenceBackendUnavailable(
        f"{what}: the reference (pure-MLX, CPU) backend is not part of this library; "
        "use backend='cuda' (or 'auto' / the Metal names, which all select the CUDA kernels)"
    )
