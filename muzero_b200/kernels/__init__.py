from .loader import (
    load_mu_zero_cuda_extension,
    mu_zero_quantize_cuda,
    mu_zero_dequantize_cuda,
    mu_zero_qk_cuda,
    mu_zero_av_cuda,
)
from ._cabi import MuZeroKernelError

__all__ = [
    "load_mu_zero_cuda_extension",
    "mu_zero_quantize_cuda",
    "mu_zero_dequantize_cuda",
    "mu_zero_qk_cuda",
    "mu_zero_av_cuda",
    "MuZeroKernelError",
]
