"""Quantizer front end: alpha selection and flat-row quantize / dequantize.

Mirrors the public functions of the reference's ``muzero/quantizer.py``
(``select_alpha`` :29-83, ``quantize_rows`` :119-158, ``dequantize_rows``
:205-226, ``roundtrip`` :273-323).  The row kernels are the CUDA library's; there
is no torch or Triton backend behind them, so CPU tensors raise.
Alpha selection is a one-time statistic per layer and stays in torch.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .kernels.loader import MuZeroKernelError, mu_zero_dequantize_cuda, mu_zero_quantize_cuda

_TINY = 1e-8


def alpha_from_stats(*, bits: int, kind: str, tail_ratio: float, concentration_ratio: float,
                     anchor_offset: float) -> float:
    """Decision table of the reference (muzero/quantizer.py:65-83)."""
    if kind == "key":
        if bits == 1:
            if tail_ratio > 3.0 or concentration_ratio > 12.0 or anchor_offset > 0.22:
                return 16.0
            if tail_ratio > 2.0 or concentration_ratio > 8.0 or anchor_offset > 0.16:
                return 4.0
            return 2.0
        if bits == 8 and (tail_ratio > 2.6 or concentration_ratio > 10.0):
            return 4.0
        return 2.0
    if bits >= 8:
        if tail_ratio > 2.0 or concentration_ratio > 6.0 or anchor_offset > 0.14:
            return 4.0
        return 2.0
    if bits == 3 and tail_ratio > 2.3 and anchor_offset > 0.12:
        return 4.0
    return 2.0


def _magnitude_ratios(sample: torch.Tensor) -> tuple[float, float]:
    """(p99/p95, p95/p50) of |sample| by order statistics at k = max(1, floor(p*n))."""
    mag = sample.float().abs().reshape(-1)
    n = mag.numel()
    ks = [max(1, int(p * n)) for p in (0.50, 0.95, 0.99)]
    ordered, _ = torch.sort(mag)
    p50, p95, p99 = (float(v) for v in ordered[torch.tensor(ks, device=mag.device) - 1].tolist())
    return p99 / max(p95, _TINY), p95 / max(p50, _TINY)


def _strided_sample(flat: torch.Tensor, max_points: int) -> torch.Tensor:
    if flat.numel() <= max_points:
        return flat
    step = max(1, flat.numel() // max_points)
    return flat[::step][:max_points]


def _anchor_offset(groups: torch.Tensor) -> float:
    """mean |zero_anchor - 0.5| over groups laid out on the last axis."""
    lo = groups.amin(dim=-1)
    hi = groups.amax(dim=-1)
    anchor = ((0.0 - lo) / (hi - lo).clamp_min(_TINY)).clamp(0.0, 1.0)
    return float((anchor - 0.5).abs().mean())


def select_alpha(tensor: torch.Tensor, *, bits: int, q_group_size: int, kind: str,
                 max_points: int = 65536) -> float:
    """Log-compander alpha for ``tensor`` ([N,G] rows or [B,H,S,D]); always 2.0 for 4 bits."""
    if bits == 4:
        return 2.0
    work = tensor.float()
    tail, conc = _magnitude_ratios(_strided_sample(work.reshape(-1), max_points))
    if work.dim() == 2:
        rows, width = work.shape
        if width != q_group_size:
            ng = max(1, width // q_group_size)
            work = work[:, : ng * q_group_size].reshape(rows, ng, q_group_size)
    else:
        if kind == "key":
            work = work.transpose(2, 3).contiguous()
        b, h, s, d = work.shape
        d_pad = -(-d // q_group_size) * q_group_size
        if d_pad != d:
            work = F.pad(work, (0, d_pad - d))
        work = work.reshape(b, h, s, d_pad // q_group_size, q_group_size)
    return alpha_from_stats(bits=bits, kind=kind, tail_ratio=tail, concentration_ratio=conc,
                            anchor_offset=_anchor_offset(work))


def select_alpha_key_block(block: torch.Tensor, *, bits: int, q_group_size: int, max_points: int = 65536) -> float:
    """``select_alpha(rows, kind="key")`` for the rows [B*KVH*nsg*D, G] of a key block
    [B,KVH,nsg*G,D], without materialising the transposed rows: the strided sample is
    gathered through the row index arithmetic and the group min/max reduce over the token axis.
    """
    if bits == 4:
        return 2.0
    b, h, s, d = block.shape
    g = q_group_size
    nsg = s // g
    total = b * h * nsg * d * g
    step = max(1, total // max_points) if total > max_points else 1
    idx = torch.arange(0, total, step, device=block.device)[:max_points] if total > max_points \
        else torch.arange(0, total, device=block.device)
    t = idx % g
    rest = idx // g
    ch = rest % d
    rest = rest // d
    grp = rest % nsg
    rest = rest // nsg
    hh = rest % h
    bb = rest // h
    sample = block[bb, hh, grp * g + t, ch]
    tail, conc = _magnitude_ratios(sample)
    grouped = block[:, :, : nsg * g].float().reshape(b, h, nsg, g, d).transpose(3, 4)
    return alpha_from_stats(bits=bits, kind="key", tail_ratio=tail, concentration_ratio=conc,
                            anchor_offset=_anchor_offset(grouped))


def quantize_rows(flat_grouped: torch.Tensor, bits: int, alpha: float, amax_eps: float,
                  amax_dtype: torch.dtype, *, backend: str = "auto", _cuda_ok: bool = True,
                  _triton_ok: bool = True):
    """[N,G] -> (packed uint8 [N,QB], mn [N,1], scale [N,1]).  ``backend`` is ignored."""
    if not flat_grouped.is_cuda:
        raise MuZeroKernelError("quantize_rows needs a CUDA tensor; this package has no CPU path")
    n, g = flat_grouped.shape
    qb = (g * bits + 7) // 8
    dev = flat_grouped.device
    packed = torch.empty((n, qb), dtype=torch.uint8, device=dev)
    mn = torch.empty((n, 1), dtype=amax_dtype, device=dev)
    scale = torch.empty((n, 1), dtype=amax_dtype, device=dev)
    mu_zero_quantize_cuda(flat_grouped.contiguous(), packed, mn, scale, bits, float(alpha), amax_eps)
    return packed, mn, scale


def dequantize_rows(packed_q: torch.Tensor, mn: torch.Tensor, scale: torch.Tensor, bits: int, alpha: float,
                    q_group_size: int, out_dtype: torch.dtype, *, amax_eps: float = 1e-8,
                    _cuda_ok: bool = True) -> torch.Tensor:
    """Inverse of ``quantize_rows``: [N,QB] -> [N,G] in ``out_dtype``."""
    if not packed_q.is_cuda:
        raise MuZeroKernelError("dequantize_rows needs CUDA tensors; this package has no CPU path")
    out = torch.empty((packed_q.shape[0], q_group_size), dtype=out_dtype, device=packed_q.device)
    mu_zero_dequantize_cuda(packed_q.contiguous(), mn.contiguous(), scale.contiguous(), out, bits, float(alpha), amax_eps)
    return out


def roundtrip(key: torch.Tensor, value: torch.Tensor, *, bits: int = 4, q_group_size: int = 64,
              alpha_key: Optional[float] = None, alpha_value: Optional[float] = None,
              amax_dtype: torch.dtype = torch.float16, amax_eps: float = 1e-8):
    """Quantize then dequantize K ([B,H,S,D], grouped over tokens) and V (grouped over channels)."""
    g = q_group_size
    if alpha_key is None:
        alpha_key = select_alpha(key, bits=bits, q_group_size=g, kind="key")
    if alpha_value is None:
        alpha_value = select_alpha(value, bits=bits, q_group_size=g, kind="value")

    b, h, s, d = key.shape
    nsg = s // g
    rows = key.reshape(b, h, nsg, g, d).transpose(3, 4).contiguous().reshape(-1, g).float()
    back = dequantize_rows(*quantize_rows(rows, bits, alpha_key, amax_eps, amax_dtype), bits, alpha_key, g,
                           key.dtype, amax_eps=amax_eps)
    key_out = back.reshape(b, h, nsg, d, g).transpose(3, 4).reshape(b, h, s, d).contiguous()

    b, h, s, d = value.shape
    d_pad = -(-d // g) * g
    padded = F.pad(value, (0, d_pad - d)) if d_pad != d else value
    rows = padded.reshape(-1, g).float()
    back = dequantize_rows(*quantize_rows(rows, bits, alpha_value, amax_eps, amax_dtype), bits, alpha_value, g,
                           value.dtype, amax_eps=amax_eps)
    value_out = back.reshape(b, h, s, d_pad)[..., :d].contiguous()
    return key_out, value_out
