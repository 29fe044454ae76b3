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


def gather_partials(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor,
                    group: Optional[dist.ProcessGroup] = None):
    """All-gathers one rank's (m[B,H], l[B,H], acc[B,H,D]) into stacked [world, ...] tensors.

    The three tensors travel as one buffer [B,H,D+2] so that a decode step costs one collective."""
    world = dist.get_world_size(group)
    packed = torch.cat([acc, m.unsqueeze(-1), l.unsqueeze(-1)], dim=-1).contiguous()
    flat = torch.empty((world * packed.shape[0], *packed.shape[1:]), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(flat, packed, group=group)
    out = flat.view(world, *packed.shape)
    d = acc.shape[-1]
    return out[..., d].contiguous(), out[..., d + 1].contiguous(), out[..., :d].contiguous()


def kv_split_decode_attention(layer, query: torch.Tensor, scaling: float, *, out_dtype: Optional[torch.dtype] = None,
                              group: Optional[dist.ProcessGroup] = None,
                              partial_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None) -> torch.Tensor:
    """Decode attention when ``layer`` holds only this rank's slice of the sequence.

    Every rank gets the full result [B,1,H,D].  ``partial_fn`` / ``merge_fn`` default to the CUDA
    entry points (``mz_decode_attention_partial`` / ``mz_lse_merge``); tests of the host logic on
    CPU ranks substitute CPU functions."""
    if partial_fn is None or merge_fn is None:
        from .cache.attention import decode_attention_partial, lse_merge
        partial_fn = partial_fn or decode_attention_partial
        merge_fn = merge_fn or lse_merge
    m, l, acc = partial_fn(layer, query, scaling)
    ms, ls, accs = gather_partials(m, l, acc, group)
    return merge_fn(ms, ls, accs, out_dtype or query.dtype)
