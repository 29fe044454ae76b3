"""``MuZeroConfig``: settings of the quantized KV cache.

Same fields, defaults and validation as the reference's dataclass
(muzero/config.py:7-51) so that ``cache_config`` dictionaries written for the
reference keep working.  ``backend`` is accepted for compatibility only: this
package has a single execution path (the sm_100a CUDA library), so every
accepted value selects it.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Optional

SUPPORTED_BITS = (1, 2, 3, 4, 7, 8)
SUPPORTED_META_DTYPES = ("float16", "bfloat16", "float32")
ACCEPTED_BACKENDS = ("auto", "cuda", "triton", "torch")


@dataclass
class MuZeroConfig:
    bits: int = 4                       # code width; the cache accepts 1,2,3,4,7,8 (kernels handle 1..8)
    q_group_size: int = 64              # values per quantization group
    residual_length: int = 128          # newest tokens kept in full precision
    amax_dtype: str = "float16"         # storage type of the per-group (min, range) metadata
    stats_max_points: int = 65536       # sample size of the alpha statistics
    backend: str = "auto"               # accepted for compatibility; always the CUDA library
    alpha_key: Optional[float] = None   # None = choose at first flush
    alpha_value: Optional[float] = None
    logq_compatible_layout: bool = False
    decode_flush_by_group: bool = True  # flush every q_group_size decode steps (else every 4 groups)

    def __post_init__(self) -> None:
        problems = []
        if self.bits not in SUPPORTED_BITS:
            problems.append(f"`bits` must be one of {set(SUPPORTED_BITS)}, got {self.bits}")
        if self.q_group_size <= 0:
            problems.append(f"`q_group_size` must be > 0, got {self.q_group_size}")
        if self.amax_dtype not in SUPPORTED_META_DTYPES:
            problems.append(f"`amax_dtype` must be one of {set(SUPPORTED_META_DTYPES)}, got {self.amax_dtype}")
        if self.backend not in ACCEPTED_BACKENDS:
            problems.append(f"`backend` must be one of {set(ACCEPTED_BACKENDS)}, got {self.backend}")
        if (not problems and self.decode_flush_by_group
                and self.residual_length % self.q_group_size != 0):
            problems.append("`residual_length` must be a multiple of `q_group_size` when `decode_flush_by_group=True`")
        if problems:
            raise ValueError("; ".join(problems))

    @classmethod
    def from_dict(cls, d: dict) -> "MuZeroConfig":
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})
