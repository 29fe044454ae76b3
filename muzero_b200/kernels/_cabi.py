"""ctypes binding of ``libmuzero_b200.so`` (declared in ``include/muzero_b200.h``).

There is no fallback: if the shared library is missing or a call returns a
non-zero status this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_longlong, c_size_t, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MUZERO_B200_LIB") or os.path.join(os.path.dirname(_HERE), "lib", "libmuzero_b200.so")

MZ_F32, MZ_F16, MZ_BF16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: MZ_F32, torch.float16: MZ_F16, torch.bfloat16: MZ_BF16}

# every symbol the public header declares
EXPORTS = (
    "mz_version", "mz_last_error", "mz_set_expand_table", "mz_quantize_rows", "mz_dequantize_rows",
    "mz_flush_kv", "mz_append_kv", "mz_dequantize_kv", "mz_decode_workspace_bytes", "mz_decode_attention",
    "mz_decode_attention_partial", "mz_lse_merge", "mz_qk_logits", "mz_av_output", "mz_decode_attention_static",
    "mz_decode_step", "mz_decode_step_workspace_bytes", "mz_flush_kv_parts", "mz_decode_workspace_bound", "mz_decode_attention_partial_packed", "mz_lse_merge_packed", "mz_store_gather_batch", "mz_debug_force_kernel", "mz_bounds_violations",
)


class MuZeroKernelError(RuntimeError):
    pass


class KVStore(Structure):
    _fields_ = [
        ("batch", c_int), ("kv_heads", c_int), ("head_dim", c_int),
        ("group", c_int), ("bits", c_int),
        ("meta_dtype", c_int), ("kv_dtype", c_int),
        ("alpha_key", c_float), ("alpha_value", c_float),
        ("packed_k", c_void_p), ("k_mn", c_void_p), ("k_scale", c_void_p),
        ("pk_stride_b", c_longlong), ("pk_stride_h", c_longlong), ("km_stride_b", c_longlong), ("km_stride_h", c_longlong),
        ("packed_v", c_void_p), ("v_mn", c_void_p), ("v_scale", c_void_p),
        ("pv_stride_b", c_longlong), ("pv_stride_h", c_longlong), ("vm_stride_b", c_longlong), ("vm_stride_h", c_longlong),
        ("k_groups", c_int), ("v_tokens", c_int),
        ("res_k", c_void_p), ("res_v", c_void_p),
        ("res_stride_b", c_longlong), ("res_stride_h", c_longlong), ("res_stride_t", c_longlong),
        ("res_start", c_int), ("res_len", c_int),
    ]


class DecodeArgs(Structure):
    _fields_ = [
        ("store", KVStore),
        ("q_heads", c_int),
        ("query", c_void_p),
        ("q_stride_b", c_longlong), ("q_stride_h", c_longlong),
        ("scaling", c_float),
        ("mask", c_void_p),
        ("mask_dtype", c_int),
        ("mask_stride_b", c_longlong),
        ("out", c_void_p),
        ("out_dtype", c_int),
        ("splits", c_int),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
    ]


_lib = None


def load_library() -> ctypes.CDLL:
    """Loads the CUDA library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise MuZeroKernelError(
            f"{LIB_PATH} is missing: build it with `python -m muzero_b200.build` (needs nvcc); "
            "there is no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    missing = [s for s in EXPORTS if not hasattr(lib, s)]
    if missing:
        raise MuZeroKernelError(f"{LIB_PATH} lacks symbols {missing}; rebuild it")
    lib.mz_version.restype = c_int
    lib.mz_last_error.argtypes = [c_char_p, c_int]
    lib.mz_set_expand_table.argtypes = [c_int, c_float, c_void_p]
    lib.mz_quantize_rows.argtypes = [c_void_p, c_int, c_longlong, c_int, c_int, c_float, c_float, c_void_p, c_void_p,
                                     c_void_p, c_int, c_void_p]
    lib.mz_dequantize_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_float, c_float,
                                       c_void_p, c_int, c_void_p]
    lib.mz_flush_kv.argtypes = [POINTER(KVStore), c_int, c_float, c_void_p]
    lib.mz_flush_kv_parts.argtypes = [POINTER(KVStore), c_int, c_int, c_int, c_float, c_void_p]
    lib.mz_append_kv.argtypes = [POINTER(KVStore), c_void_p, c_void_p, c_longlong, c_longlong, c_void_p]
    lib.mz_dequantize_kv.argtypes = [POINTER(KVStore), c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_float, c_void_p]
    lib.mz_decode_workspace_bytes.argtypes = [POINTER(DecodeArgs)]
    lib.mz_decode_workspace_bytes.restype = c_size_t
    lib.mz_decode_workspace_bound.argtypes = [POINTER(DecodeArgs)]
    lib.mz_decode_workspace_bound.restype = c_size_t
    lib.mz_decode_attention.argtypes = [POINTER(DecodeArgs), c_void_p]
    lib.mz_decode_attention_static.argtypes = [POINTER(DecodeArgs), c_void_p]
    lib.mz_decode_step.argtypes = [POINTER(DecodeArgs), c_void_p, c_void_p, c_longlong, c_longlong, c_int, c_int, c_int, c_int,
                                   c_float, c_void_p]
    lib.mz_decode_step_workspace_bytes.argtypes = [POINTER(DecodeArgs), c_int, c_int]
    lib.mz_decode_step_workspace_bytes.restype = c_size_t
    lib.mz_decode_attention_partial.argtypes = [POINTER(DecodeArgs), c_void_p, c_void_p, c_void_p, c_void_p]
    lib.mz_lse_merge.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_int, c_void_p, c_int, c_void_p]
    lib.mz_decode_attention_partial_packed.argtypes = [POINTER(DecodeArgs), c_void_p, c_void_p]
    lib.mz_lse_merge_packed.argtypes = [c_void_p, c_int, c_longlong, c_int, c_void_p, c_int, c_void_p]
    lib.mz_store_gather_batch.argtypes = [POINTER(KVStore), POINTER(KVStore), c_void_p, c_void_p, c_void_p]
    lib.mz_debug_force_kernel.argtypes = [c_int]
    lib.mz_debug_force_kernel.restype = c_int
    lib.mz_bounds_violations.argtypes = [ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(c_int), c_int]
    lib.mz_bounds_violations.restype = ctypes.c_longlong
    lib.mz_qk_logits.argtypes = [POINTER(KVStore), c_void_p, c_longlong, c_longlong, c_int, c_float, c_void_p, c_int, c_void_p]
    lib.mz_av_output.argtypes = [POINTER(KVStore), c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
    _lib = lib
    return lib


def last_error() -> str:
    buf = ctypes.create_string_buffer(512)
    load_library().mz_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    if status != 0:
        raise MuZeroKernelError(f"{what} failed (status {status}): {last_error()}")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise MuZeroKernelError(f"unsupported dtype {dt}") from None


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise MuZeroKernelError("muzero_b200 kernels need CUDA tensors; there is no CPU path")
