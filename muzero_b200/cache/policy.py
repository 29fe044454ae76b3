"""Pure host arithmetic of the cache: flush policy and buffer capacities.

Kept free of device work so that it can be tested without a GPU.
Reference: muzero/cache/layer.py:135-169 (residual capacity rule) and
:369-401 (how many of the oldest residual tokens a flush takes).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class FlushPlan:
    key_tokens: int     # oldest residual key tokens to quantize (multiple of the group size)
    value_tokens: int   # oldest residual value tokens to quantize


def plan_flush(*, key_len: int, value_len: int, residual_length: int, group: int, decode_flush: bool,
               flush_by_group: bool, logq_layout: bool) -> FlushPlan:
    """How much of the residual window moves into the quantized store.

    Keys flush in whole units: one group, or four groups for single-token
    updates when neither ``flush_by_group`` nor ``logq_layout`` is set.  Values
    follow the keys, except in ``logq_layout`` where every value token beyond
    the residual length is flushed.
    """
    unit = group
    if decode_flush and not (logq_layout or flush_by_group):
        unit = 4 * group
    key_tokens = (max(key_len - residual_length, 0) // unit) * unit
    if logq_layout:
        value_tokens = max(value_len - residual_length, 0)
    else:
        value_tokens = min(key_tokens, value_len)
    return FlushPlan(key_tokens, value_tokens)


def residual_capacity(min_tokens: int, residual_length: int, group: int) -> int:
    """Capacity (tokens) of the residual buffer: room for the window plus two flush
    units of 4 groups, rounded up to that unit, so that the window can slide for many
    steps before it has to be moved back to the front."""
    unit = 4 * group
    need = max(min_tokens, residual_length + unit) + unit
    return -(-need // unit) * unit


def grown_capacity(current: int, needed: int, slack: int = 8) -> int:
    """Capacity of the quantized store (key groups or value tokens) after growth.

    The first allocation is the need plus one eighth (at least ``slack``), so a
    prefill followed by a few hundred decode steps fits without a copy and
    without doubling the footprint; later growth is by half.
    """
    if needed <= current:
        return current
    if current == 0:
        return needed + max(slack, needed // 8)
    return max(needed, current + max(slack, current // 2))
