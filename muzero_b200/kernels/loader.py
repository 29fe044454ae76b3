"""Python entry points of the CUDA library, under the names the reference's
``muzero.kernels`` exposes (muzero/kernels/loader.py:1862-1911): same argument
order and meaning, caller-allocated outputs, launch on torch's current stream.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _cabi
from ._cabi import KVStore, MuZeroKernelError, check, dtype_code, require_cuda, stream_ptr

_tables_installed: set = set()


def load_mu_zero_cuda_extension():
    """Returns the loaded C-ABI library; raises if it was not built."""
    return _cabi.load_library()


def expand_table_host(bits: int, alpha: float) -> torch.Tensor:
    """fp32 table [2^bits, 2^bits] of the compander inverse, computed with torch CPU ops.

    Entry [denom, numer] = expm1(clamp(numer/denom, 0, 1) * log1p(alpha)) / alpha — the
    values the reference's torch dequantizer produces (muzero/quantizer.py:249-253), so a
    dequantizer that reads them is bit-identical to it.
    """
    top = (1 << bits) - 1
    log_base = torch.log1p(torch.tensor(float(alpha), dtype=torch.float32))
    denom = torch.arange(0, top + 1, dtype=torch.float32).clamp_min(1.0).unsqueeze(1)
    numer = torch.arange(0, top + 1, dtype=torch.float32).unsqueeze(0)
    return (torch.expm1((numer / denom).clamp(0.0, 1.0) * log_base) / float(alpha)).contiguous()


def ensure_expand_table(bits: int, alpha: float, device: torch.device) -> None:
    """Installs torch's table for (bits, alpha) on ``device`` once per process."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, int(bits), float(alpha))
    if key in _tables_installed:
        return
    table = expand_table_host(bits, alpha)
    with torch.cuda.device(index):
        check(load_mu_zero_cuda_extension().mz_set_expand_table(int(bits), float(alpha), table.data_ptr()),
              "mz_set_expand_table")
    _tables_installed.add(key)


def _contig(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_contiguous():
        raise MuZeroKernelError(f"{name} must be contiguous")
    return t


def mu_zero_quantize_cuda(grouped, packed_q, mn, scale, bits, alpha, eps):
    """grouped[N,G] -> packed_q[N,QB] u8, mn[N,1], scale[N,1] (all caller allocated)."""
    require_cuda(grouped, packed_q, mn, scale)
    n, g = grouped.shape
    lib = load_mu_zero_cuda_extension()
    with torch.cuda.device(grouped.device):
        check(lib.mz_quantize_rows(_contig(grouped, "grouped").data_ptr(), dtype_code(grouped.dtype), n, g, int(bits),
                                   float(alpha), float(eps), _contig(packed_q, "packed_q").data_ptr(),
                                   _contig(mn, "mn").data_ptr(), _contig(scale, "scale").data_ptr(),
                                   dtype_code(mn.dtype), stream_ptr(grouped.device)), "mz_quantize_rows")


def mu_zero_dequantize_cuda(packed_q, mn, scale, output, bits, alpha, eps: float = 1e-8):
    """packed_q[N,QB], mn[N,1], scale[N,1] -> output[N,G] (caller allocated)."""
    require_cuda(packed_q, mn, scale, output)
    n, g = output.shape
    lib = load_mu_zero_cuda_extension()
    ensure_expand_table(bits, alpha, packed_q.device)
    with torch.cuda.device(packed_q.device):
        check(lib.mz_dequantize_rows(_contig(packed_q, "packed_q").data_ptr(), _contig(mn, "mn").data_ptr(),
                                     _contig(scale, "scale").data_ptr(), dtype_code(mn.dtype), n, g, int(bits),
                                     float(alpha), float(eps), _contig(output, "output").data_ptr(),
                                     dtype_code(output.dtype), stream_ptr(packed_q.device)), "mz_dequantize_rows")


def _prefix_store(packed_q, mn, scale, bits, alpha, kind: str, group_size: Optional[int], kv_dtype) -> KVStore:
    """A store descriptor that holds only a key prefix or only a value prefix."""
    s = KVStore()
    b, kvh = packed_q.shape[0], packed_q.shape[1]
    s.batch, s.kv_heads, s.bits = b, kvh, int(bits)
    s.meta_dtype, s.kv_dtype = dtype_code(mn.dtype), dtype_code(kv_dtype)
    s.alpha_key = s.alpha_value = float(alpha)
    qb = packed_q.shape[-1]
    if kind == "key":       # [B,KVH,NSG,D,QB]
        s.head_dim = packed_q.shape[3]
        s.group = group_size if group_size is not None else (qb * 8) // int(bits)
        s.k_groups = packed_q.shape[2]
        s.packed_k, s.k_mn, s.k_scale = packed_q.data_ptr(), mn.data_ptr(), scale.data_ptr()
        s.pk_stride_b, s.pk_stride_h = packed_q.stride(0), packed_q.stride(1)
        s.km_stride_b, s.km_stride_h = mn.stride(0), mn.stride(1)
        s.packed_v, s.v_mn, s.v_scale = s.packed_k, s.k_mn, s.k_scale
    else:                   # [B,KVH,S,NG,QB]
        s.group = int(group_size)
        s.head_dim = packed_q.shape[3] * s.group
        s.v_tokens = packed_q.shape[2]
        s.packed_v, s.v_mn, s.v_scale = packed_q.data_ptr(), mn.data_ptr(), scale.data_ptr()
        s.pv_stride_b, s.pv_stride_h = packed_q.stride(0), packed_q.stride(1)
        s.vm_stride_b, s.vm_stride_h = mn.stride(0), mn.stride(1)
        s.packed_k, s.k_mn, s.k_scale = s.packed_v, s.v_mn, s.v_scale
    return s


def mu_zero_qk_cuda(query, packed_q, mn, scale, output, bits, alpha, num_key_value_groups, scaling):
    """query[B,H,1,D], key store [B,KVH,NSG,D,QB] -> output[B,H,NSG*G] scaled logits."""
    require_cuda(query, packed_q, mn, scale, output)
    for t, nm in ((packed_q, "packed_q"), (mn, "mn"), (scale, "scale"), (output, "output")):
        _contig(t, nm)
    if query.stride(-1) != 1:
        raise MuZeroKernelError("query must be contiguous in its last dimension")
    group = output.shape[-1] // max(packed_q.shape[2], 1) if packed_q.shape[2] else None
    store = _prefix_store(packed_q, mn, scale, bits, alpha, "key", group, query.dtype)
    ensure_expand_table(bits, alpha, query.device)
    with torch.cuda.device(query.device):
        check(load_mu_zero_cuda_extension().mz_qk_logits(
            ctypes.byref(store), query.data_ptr(), query.stride(0), query.stride(1), query.shape[1], float(scaling),
            output.data_ptr(), dtype_code(output.dtype), stream_ptr(query.device)), "mz_qk_logits")


def mu_zero_av_cuda(attn_weights, packed_q, mn, scale, output, bits, alpha, num_key_value_groups, group_size):
    """attn_weights[B,H,S], value store [B,KVH,S,NG,QB] -> output[B,H,D]."""
    require_cuda(attn_weights, packed_q, mn, scale, output)
    for t, nm in ((attn_weights, "attn_weights"), (packed_q, "packed_q"), (mn, "mn"), (scale, "scale"), (output, "output")):
        _contig(t, nm)
    store = _prefix_store(packed_q, mn, scale, bits, alpha, "value", group_size, output.dtype if output.dtype != torch.float32 else torch.bfloat16)
    if output.shape[-1] > store.head_dim:
        raise MuZeroKernelError("output head_dim exceeds the stored value width")
    store.head_dim = output.shape[-1]
    ensure_expand_table(bits, alpha, attn_weights.device)
    with torch.cuda.device(attn_weights.device):
        check(load_mu_zero_cuda_extension().mz_av_output(
            ctypes.byref(store), attn_weights.data_ptr(), dtype_code(attn_weights.dtype), attn_weights.shape[-1],
            attn_weights.shape[1], output.data_ptr(), dtype_code(output.dtype), stream_ptr(attn_weights.device)),
            "mz_av_output")
