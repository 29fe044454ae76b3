"""Multi-GPU modes of the hot path (one process per GPU, ``torch.distributed``).

The reference is single-GPU; these are the two ways its path shards:

* **batch sharding** — sequences never interact (every reference kernel indexes the batch
  independently, e.g. muzero/kernels/loader.py:574-577,916-918), so each rank owns a slice of
  the batch and there is no data-path collective;
* **KV-sequence split** — softmax over a partition of the keys composes by log-sum-exp, which
  the reference already uses across chunks on one GPU (muzero/kernels/loader.py:1249-1285,
  muzero/cache/attention.py:153-169).  Rank r holds a contiguous slice of the tokens, computes
  the partial (m, l, acc) triple of its slice, the triples are all-gathered into local memory
  and merged locally.  This is the only collective on the path (B*H*(D+2) floats per rank).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def batch_shard(total_batch: int, rank: int, world: int) -> slice:
    """Contiguous, balanced slice of the batch owned by ``rank`` (sizes differ by at most one)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total_batch, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def kv_split_ranges(total_tokens: int, world: int, group: int) -> list[tuple[int, int]]:
    """Token ranges [start, end) per rank, cut at multiples of ``group`` (quantization groups are
    never split); the last rank takes the remainder, i.e. the newest tokens and the residual window."""
    groups = total_tokens // group
    base, extra = divmod(groups, world)
    out, start = [], 0
    for r in range(world):
        n = (base + (1 if r < extra else 0)) * group
        end = total_tokens if r == world - 1 else start + n
        out.append((start, end))
        start = end
    return out


def pack_partial(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor) -> torch.Tensor:
    """(m[B,H], l[B,H], acc[B,H,D]) -> one record tensor [B,H,D+2] = {acc, m, l}."""
    return torch.cat([acc, m.unsqueeze(-1), l.unsqueeze(-1)], dim=-1).contiguous()


def unpack_partials(records: torch.Tensor):
    """[...,D+2] records -> views (m, l, acc)."""
    d = records.shape[-1] - 2
    return records[..., d], records[..., d + 1], records[..., :d]


_gather_buffers: dict = {}


def gather_records(record: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gathers one rank's packed record [B,H,D+2] into [world,B,H,D+2]: the one collective of a decode
    step, into a buffer kept per (device, shape, world)."""
    world = dist.get_world_size(group)
    key = (record.device, tuple(record.shape), world)
    flat = _gather_buffers.get(key)
    if flat is None:
        flat = torch.empty((world, *record.shape), dtype=record.dtype, device=record.device)
        _gather_buffers[key] = flat
    # the collective sees the ranks' records concatenated along the first dimension
    dist.all_gather_into_tensor(flat.view(world * record.shape[0], *record.shape[1:]), record, group=group)
    return flat


def kv_split_decode_attention(layer, query: torch.Tensor, scaling: float, *, out_dtype: Optional[torch.dtype] = None,
                              group: Optional[dist.ProcessGroup] = None,
                              record_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None) -> torch.Tensor:
    """Decode attention when ``layer`` holds only this rank's slice of the sequence.

    Every rank gets the full result [B,1,H,D].  Three launches per call: the partial kernel writes this rank's
    packed record, NCCL all-gathers the records into local memory, the merge kernel reads them with a stride.
    ``record_fn(layer, query, scaling) -> [B,H,D+2]`` and ``merge_fn(records[world,B,H,D+2], dtype)`` default to
    the CUDA entry points (``mz_decode_attention_partial_packed`` / ``mz_lse_merge_packed``); tests of the host
    logic on CPU ranks substitute CPU functions."""
    if record_fn is None or merge_fn is None:
        from .cache.attention import decode_attention_partial_packed, lse_merge_packed
        record_fn = record_fn or decode_attention_partial_packed
        merge_fn = merge_fn or lse_merge_packed
    records = gather_records(record_fn(layer, query, scaling), group)
    return merge_fn(records, out_dtype or query.dtype)
