"""muzero_b200: the muZero KV-cache hot path (quantizer, residual-window flush, quantized
decode attention) as hand-written sm_100a CUDA behind the reference's plug-in API.

    import muzero_b200 as muzero
    muzero.patch_transformers()
    model.generate(..., cache_implementation="mu_zero_4bit",
                   cache_config={"q_group_size": 64, "residual_length": 128})
"""
from .config import MuZeroConfig
from .quantizer import select_alpha, quantize_rows, dequantize_rows, roundtrip
from .cache.layer import MuZeroCacheLayer
from .cache.attention import get_mu_zero_decode_stats, mu_zero_decode_attention_forward, reset_mu_zero_decode_stats
from .integrations.transformers_patch import MuZeroCache, patch_transformers

__all__ = [
    "MuZeroConfig",
    "MuZeroCacheLayer",
    "MuZeroCache",
    "select_alpha",
    "quantize_rows",
    "dequantize_rows",
    "roundtrip",
    "mu_zero_decode_attention_forward",
    "reset_mu_zero_decode_stats",
    "get_mu_zero_decode_stats",
    "patch_transformers",
]

__version__ = "0.1.0"
