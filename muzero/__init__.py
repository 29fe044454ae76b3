"""Drop-in alias: ``import muzero`` resolves to ``muzero_b200`` (same public names and
sub-module paths as the reference package), so code written against the reference runs
unchanged on the B200 implementation."""
import importlib
import sys

import muzero_b200 as _impl
from muzero_b200 import *  # noqa: F401,F403
from muzero_b200 import __all__, __version__  # noqa: F401

for _name in ("config", "quantizer", "cache", "cache.layer", "cache.attention", "kernels", "kernels.loader",
              "integrations", "integrations.transformers_patch"):
    sys.modules[f"{__name__}.{_name}"] = importlib.import_module(f"muzero_b200.{_name}")
