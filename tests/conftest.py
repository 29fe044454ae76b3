"""Shared fixtures: marker registration, oracle loader, golden readers."""
import hashlib
import importlib.util
import json
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_oracle():
    """The CPU oracle lives outside the package on purpose; load it by path."""
    name = "mz_oracle"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "oracle", "mz_oracle.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def oracle():
    return load_oracle()


@pytest.fixture(scope="session")
def golden():
    class G:
        rows_quant = np.load(os.path.join(GOLDEN, "rows_quant.npz"))
        rows_dequant = np.load(os.path.join(GOLDEN, "rows_dequant.npz"))
        tables = np.load(os.path.join(GOLDEN, "expand_tables.npz"))
        layer = np.load(os.path.join(GOLDEN, "layer_cases.npz"))
        layer_meta = json.load(open(os.path.join(GOLDEN, "layer_cases.json")))
        layer_logq = np.load(os.path.join(GOLDEN, "layer_cases_logq.npz"))
        layer_logq_meta = json.load(open(os.path.join(GOLDEN, "layer_cases_logq.json")))
        config0 = np.load(os.path.join(GOLDEN, "config0.npz"))
        config0_meta = json.load(open(os.path.join(GOLDEN, "config0.json")))
        alpha = json.load(open(os.path.join(GOLDEN, "alpha_cases.json")))
    return G


def sha(t: torch.Tensor) -> str:
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.view(torch.int16)
    return hashlib.sha256(t.numpy().tobytes()).hexdigest()


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().cpu().view(torch.int16).numpy().view(np.uint16)


def from_bits16(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(dtype)


DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
