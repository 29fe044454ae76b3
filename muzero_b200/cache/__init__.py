from .layer import MuZeroCacheLayer
from .attention import mu_zero_decode_attention_forward

__all__ = ["MuZeroCacheLayer", "mu_zero_decode_attention_forward"]
