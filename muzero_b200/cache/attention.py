"""Decode-step attention over the quantized cache: one fused CUDA call.

Same call contract as the reference's ``mu_zero_decode_attention_forward``
(muzero/cache/attention.py:48-295): returns ``(attn_output [B,1,H,D], None)`` for a
single-token query, ``None`` when the caller should run its stock attention
(multi-token query or no cache layer), and counts calls in the statistics the
reference's benchmark reads.  Where the reference launches a QK kernel, torch
matmuls for the residual, a concatenation, a softmax, an AV kernel and an add,
this module makes a single C-ABI call that covers packed prefix and residual.
"""
from __future__ import annotations

import ctypes
from collections import defaultdict
from typing import Optional

import torch

from ..kernels._cabi import DecodeArgs, MuZeroKernelError, check, dtype_code, last_error, stream_ptr
from ..kernels.loader import load_mu_zero_cuda_extension

_MU_ZERO_DECODE_STATS = defaultdict(int)
_workspaces: dict = {}


def reset_mu_zero_decode_stats() -> None:
    _MU_ZERO_DECODE_STATS.clear()


def get_mu_zero_decode_stats() -> dict[str, int]:
    return dict(_MU_ZERO_DECODE_STATS)


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """One reusable scratch buffer per (device, stream); grows, never shrinks."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def build_decode_args(layer, query: torch.Tensor, scaling: float, attention_mask: Optional[torch.Tensor],
                      out: Optional[torch.Tensor], *, splits: int = 0, step: Optional[tuple[int, int]] = None,
                      bound: bool = False) -> DecodeArgs:
    """Fills the C argument block for one decode call on ``layer``.

    ``step=(residual_length, flush_unit)``: the block is for ``mz_decode_step``, i.e. the mask must
    cover one more token and the workspace is sized for the store as it will be after the step.
    ``bound=True``: the workspace is sized for any number of cached tokens (``mz_decode_workspace_bound``),
    so that the block can be reused for later steps."""
    if not query.is_cuda:
        raise MuZeroKernelError("decode attention needs CUDA tensors; this package has no CPU path")
    if query.dtype != layer.dtype:
        raise MuZeroKernelError(f"query dtype {query.dtype} differs from cache dtype {layer.dtype}")
    if query.stride(-1) != 1:
        query = query.contiguous()
    a = DecodeArgs()
    a.store = layer._store_struct()
    a.q_heads = query.shape[1]
    a.query = query.data_ptr()
    a.q_stride_b, a.q_stride_h = query.stride(0), query.stride(1)
    a.scaling = float(scaling)
    a._keepalive = [query]
    if attention_mask is not None:
        mask = attention_mask
        if mask.dtype == torch.bool:
            # the reference adds the mask tensor to the logits whatever its dtype
            mask = mask.to(query.dtype)
        if mask.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            mask = mask.to(torch.float32)
        total = a.store.k_groups * a.store.group + a.store.res_len + (1 if step else 0)
        if mask.dim() != 4 or mask.shape[1] != 1 or mask.shape[2] != 1 or mask.shape[-1] < total:
            raise MuZeroKernelError(f"attention_mask must be [B,1,1,>={total}], got {tuple(mask.shape)}")
        if mask.stride(-1) != 1:
            mask = mask.contiguous()
        a.mask = mask.data_ptr()
        a.mask_dtype = dtype_code(mask.dtype)
        a.mask_stride_b = mask.stride(0) if mask.shape[0] > 1 else 0
        a._keepalive.append(mask)
    a.splits = int(splits)
    if out is not None:
        a.out = out.data_ptr()
        a.out_dtype = dtype_code(out.dtype)
    lib = load_mu_zero_cuda_extension()
    if bound:
        need = lib.mz_decode_workspace_bound(ctypes.byref(a))
    elif step:
        need = lib.mz_decode_step_workspace_bytes(ctypes.byref(a), int(step[0]), int(step[1]))
    else:
        need = lib.mz_decode_workspace_bytes(ctypes.byref(a))
    if need == 0:   # the size query validates like the call does and leaves its message behind
        raise MuZeroKernelError(f"invalid decode-attention arguments: {last_error()}")
    ws = _workspace(query.device, need)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a._keepalive.append(ws)
    return a


def decode_attention(layer, query: torch.Tensor, scaling: float, attention_mask: Optional[torch.Tensor] = None,
                     *, out_dtype: Optional[torch.dtype] = None, splits: int = 0) -> torch.Tensor:
    """[B,H,1,D] query -> [B,1,H,D] attention output over ``layer``'s prefix + residual."""
    b, h, _, d = query.shape
    if layer._key_group_count * layer.q_group_size != layer._value_storage_len:
        # value prefix ahead of the key prefix (logq_compatible_layout): the tiled kernel reads the early values
        # from the packed store; shapes it does not serve take the two-kernel route
        kvh = layer.keys.shape[1]
        if not (d == 128 and layer.q_group_size in (32, 64, 128) and h % kvh == 0 and h // kvh in (1, 2, 4, 8)):
            return _decode_attention_unaligned(layer, query, scaling, attention_mask, out_dtype or query.dtype)
    out = torch.empty((b, 1, h, d), dtype=out_dtype or query.dtype, device=query.device)
    args = build_decode_args(layer, query, scaling, attention_mask, out, splits=splits)
    with torch.cuda.device(query.device):
        check(load_mu_zero_cuda_extension().mz_decode_attention(ctypes.byref(args), stream_ptr(query.device)),
              "mz_decode_attention")
    return out


def _decode_attention_unaligned(layer, query: torch.Tensor, scaling: float, attention_mask: Optional[torch.Tensor],
                                out_dtype: torch.dtype) -> torch.Tensor:
    """Decode attention when the value prefix is ahead of the key prefix (``logq_compatible_layout``).

    Only for shapes outside the tiled kernel (head_dim other than 128, ...): the reference's own structure
    (muzero/cache/attention.py:104-151,186-263) in fp32: packed keys through ``mz_qk_logits``, packed values
    through ``mz_av_output``, the two dense residual pieces and the softmax in torch.  Head_dim 128 caches go
    through the fused kernel, which takes the early values from the packed store."""
    from ..kernels.loader import ensure_expand_table
    if not query.is_cuda:
        raise MuZeroKernelError("decode attention needs CUDA tensors; this package has no CPU path")
    b, h, _, d = query.shape
    dev, g = query.device, layer.q_group_size
    kvh = layer.keys.shape[1]
    gqa = h // kvh
    p_k, p_v = layer._key_group_count * g, layer._value_storage_len
    lib, st, f32 = load_mu_zero_cuda_extension(), stream_ptr(dev), dtype_code(torch.float32)
    q = query if query.stride(-1) == 1 else query.contiguous()
    store = layer._store_struct()
    qg = q.float().reshape(b, kvh, gqa, d)
    pieces = []
    with torch.cuda.device(dev):
        if p_k:
            ensure_expand_table(layer.nbits, layer._selected_alpha_key, dev)
            lg = torch.empty((b, h, p_k), dtype=torch.float32, device=dev)
            check(lib.mz_qk_logits(ctypes.byref(store), q.data_ptr(), q.stride(0), q.stride(1), h, float(scaling),
                                   lg.data_ptr(), f32, st), "mz_qk_logits")
            pieces.append(lg)
        if layer.keys.shape[2]:
            pieces.append((torch.matmul(qg, layer.keys.float().transpose(-1, -2)) * scaling).reshape(b, h, -1))
        logits = torch.cat(pieces, dim=-1)
        if attention_mask is not None:
            mask = attention_mask.to(torch.float32)
            if mask.dim() != 4 or mask.shape[-1] < logits.shape[-1]:
                raise MuZeroKernelError(f"attention_mask must be [B,1,1,>={logits.shape[-1]}], got {tuple(mask.shape)}")
            logits = logits + mask[:, 0, :, : logits.shape[-1]]
        w = torch.softmax(logits, dim=-1)
        out = torch.zeros((b, h, d), dtype=torch.float32, device=dev)
        if p_v:
            ensure_expand_table(layer.nbits, layer._selected_alpha_value, dev)
            wp = w[..., :p_v].contiguous()
            check(lib.mz_av_output(ctypes.byref(store), wp.data_ptr(), f32, p_v, h, out.data_ptr(), f32, st), "mz_av_output")
        if layer.values.shape[2]:
            out = out + torch.matmul(w[..., p_v:].reshape(b, kvh, gqa, -1), layer.values.float()).reshape(b, h, d)
    return out.reshape(b, 1, h, d).to(out_dtype)


def decode_attention_reference_rounding(layer, query: torch.Tensor, scaling: float,
                                        attention_mask: Optional[torch.Tensor] = None, *, key_chunk_groups: int = 32,
                                        value_chunk_tokens: int = 256) -> torch.Tensor:
    """Parity mode: the same attention with the rounding points of the reference's torch path.

    The fused kernel keeps every intermediate in fp32.  The reference's path
    (muzero/cache/attention.py:213-239,274-290) rounds to the model dtype after the dequantization, after
    ``q K^T``, after the multiplication by ``scaling``, after the fp32 softmax, after every 256-token ``w V``
    piece and after each addition of the pieces, which moves the output by up to ~0.04.  This route repeats
    those steps on the device, op for op, with this library's bit-exact dequantizer; what still differs from
    a CPU run of the reference is the summation order inside the matmuls.  It is a debugging aid for token
    comparisons (``MUZERO_PARITY_MODE=1``), not a fast path."""
    if not query.is_cuda:
        raise MuZeroKernelError("decode attention needs CUDA tensors; this package has no CPU path")
    g, groups = layer.q_group_size, layer._key_group_count
    kvh = layer.keys.shape[1]
    rep = query.shape[1] // kvh

    def repeat_kv(x):
        return x if rep == 1 else x[:, :, None].expand(x.shape[0], kvh, rep, x.shape[2], x.shape[3]).reshape(
            x.shape[0], kvh * rep, x.shape[2], x.shape[3])

    parts, cursor = [], 0
    for sg in range(0, groups, key_chunk_groups):
        kc = repeat_kv(layer._dequantize_key_range(sg, min(sg + key_chunk_groups, groups)))
        lg = torch.matmul(query, kc.transpose(2, 3)) * scaling
        if attention_mask is not None:
            lg = lg + attention_mask[..., cursor:cursor + kc.shape[-2]]
        parts.append(lg)
        cursor += kc.shape[-2]
    dk = repeat_kv(layer.keys)
    if dk.shape[-2] > 0:
        lg = torch.matmul(query, dk.transpose(2, 3)) * scaling
        if attention_mask is not None:
            lg = lg + attention_mask[..., cursor:cursor + dk.shape[-2]]
        parts.append(lg)
    w = torch.softmax(torch.cat(parts, dim=-1), dim=-1, dtype=torch.float32).to(query.dtype)
    out, cursor = None, 0
    for st in range(0, layer._value_storage_len, value_chunk_tokens):
        vc = repeat_kv(layer._dequantize_value_range(st, min(st + value_chunk_tokens, layer._value_storage_len)))
        piece = torch.matmul(w[..., cursor:cursor + vc.shape[-2]], vc)
        out = piece if out is None else out + piece
        cursor += vc.shape[-2]
    dv = repeat_kv(layer.values)
    if dv.shape[-2] > 0:
        piece = torch.matmul(w[..., cursor:cursor + dv.shape[-2]], dv)
        out = piece if out is None else out + piece
    if out is None:
        raise MuZeroKernelError("no tokens to attend to")
    return out.transpose(1, 2).contiguous()


def decode_attention_partial(layer, query: torch.Tensor, scaling: float, attention_mask: Optional[torch.Tensor] = None,
                             *, splits: int = 0):
    """Un-normalised (m[B,H], l[B,H], acc[B,H,D]) fp32 triple of this layer's tokens."""
    b, h, _, d = query.shape
    dev = query.device
    m = torch.empty((b, h), dtype=torch.float32, device=dev)
    l = torch.empty((b, h), dtype=torch.float32, device=dev)
    acc = torch.empty((b, h, d), dtype=torch.float32, device=dev)
    args = build_decode_args(layer, query, scaling, attention_mask, None, splits=splits)
    with torch.cuda.device(dev):
        check(load_mu_zero_cuda_extension().mz_decode_attention_partial(
            ctypes.byref(args), m.data_ptr(), l.data_ptr(), acc.data_ptr(), stream_ptr(dev)), "mz_decode_attention_partial")
    return m, l, acc


def decode_attention_partial_packed(layer, query: torch.Tensor, scaling: float, attention_mask: Optional[torch.Tensor] = None,
                                    *, splits: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same triple as one packed fp32 record per row: ``[B,H,D+2]`` = ``{acc[D], m, l}`` (the unit that is
    all-gathered when the KV sequence is split over GPUs).  ``out``: write into this buffer."""
    b, h, _, d = query.shape
    rec = out if out is not None else torch.empty((b, h, d + 2), dtype=torch.float32, device=query.device)
    args = build_decode_args(layer, query, scaling, attention_mask, None, splits=splits)
    with torch.cuda.device(query.device):
        check(load_mu_zero_cuda_extension().mz_decode_attention_partial_packed(
            ctypes.byref(args), rec.data_ptr(), stream_ptr(query.device)), "mz_decode_attention_partial_packed")
    return rec


def lse_merge_packed(records: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Merges packed records stacked on dim 0 (``[P,B,H,D+2]``, contiguous) -> normalised ``[B,1,H,D]``."""
    p, b, h, dd = records.shape
    d = dd - 2
    if not records.is_contiguous():
        records = records.contiguous()
    out = torch.empty((b, 1, h, d), dtype=out_dtype, device=records.device)
    with torch.cuda.device(records.device):
        check(load_mu_zero_cuda_extension().mz_lse_merge_packed(records.data_ptr(), p, b * h, d, out.data_ptr(),
                                                                dtype_code(out_dtype), stream_ptr(records.device)),
              "mz_lse_merge_packed")
    return out


def lse_merge(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Merges partial triples stacked on dim 0 ([P,B,H], [P,B,H], [P,B,H,D]) -> [B,1,H,D]."""
    p, b, h, d = acc.shape
    out = torch.empty((b, 1, h, d), dtype=out_dtype, device=acc.device)
    m, l, acc = m.contiguous(), l.contiguous(), acc.contiguous()
    with torch.cuda.device(acc.device):
        check(load_mu_zero_cuda_extension().mz_lse_merge(m.data_ptr(), l.data_ptr(), acc.data_ptr(), p, b * h, d,
                                                         out.data_ptr(), dtype_code(out_dtype), stream_ptr(acc.device)),
              "mz_lse_merge")
    return out


def mu_zero_decode_step_forward(module, layer, key_states: torch.Tensor, value_states: torch.Tensor, query: torch.Tensor,
                                attention_mask, scaling: float):
    """The patched model forwards' decode step: ``layer.update`` of the new token followed by
    ``mu_zero_decode_attention_forward``, done by ``MuZeroCacheLayer.decode_step`` in one C call when
    the cache is in its steady state.  Returns ``(attn_output [B,1,H,D], None)`` and keeps the statistics."""
    _MU_ZERO_DECODE_STATS["calls"] += 1
    groups = getattr(module, "num_key_value_groups", None)
    if groups is not None and query.shape[1] != groups * key_states.shape[1]:
        raise MuZeroKernelError("query heads do not match num_key_value_groups * kv heads")
    out = layer.decode_step(key_states, value_states, query, scaling, attention_mask)
    if layer._key_group_count > 0:
        _MU_ZERO_DECODE_STATS["fused_qk_success"] += 1
        _MU_ZERO_DECODE_STATS["fused_av_success"] += 1
        _MU_ZERO_DECODE_STATS["fused_prefix_decode_success"] += 1
    _MU_ZERO_DECODE_STATS["returns"] += 1
    return out, None


def mu_zero_decode_attention_forward(module, query: torch.Tensor, attention_mask, scaling: float,
                                     kv_cache_state: dict, *, key_chunk_groups: int = 32,
                                     value_chunk_tokens: int = 256):
    """Attention hook for the patched model forwards; see the module docstring."""
    layer = kv_cache_state.get("layer")
    if layer is None:
        _MU_ZERO_DECODE_STATS["missing_layer"] += 1
        return None
    if query.shape[-2] != 1:
        _MU_ZERO_DECODE_STATS["non_decode_query"] += 1
        return None
    _MU_ZERO_DECODE_STATS["calls"] += 1
    groups = getattr(module, "num_key_value_groups", None)
    if groups is not None and query.shape[1] != groups * layer.keys.shape[1]:
        raise MuZeroKernelError("query heads do not match num_key_value_groups * kv heads")
    out = decode_attention(layer, query, scaling, attention_mask)
    if int(kv_cache_state.get("key_prefix_length", 0)) > 0:
        _MU_ZERO_DECODE_STATS["fused_qk_success"] += 1
        _MU_ZERO_DECODE_STATS["fused_av_success"] += 1
        _MU_ZERO_DECODE_STATS["fused_prefix_decode_success"] += 1
    _MU_ZERO_DECODE_STATS["returns"] += 1
    return out, None
