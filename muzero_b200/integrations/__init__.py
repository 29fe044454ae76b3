from .transformers_patch import patch_transformers, MuZeroCache

__all__ = ["patch_transformers", "MuZeroCache"]
