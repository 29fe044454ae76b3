"""CPU: host-side logic and the C-ABI surface (no kernel launches)."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT


def test_library_exports_every_declared_symbol():
    from muzero_b200.kernels import _cabi
    header = open(os.path.join(ROOT, "include", "muzero_b200.h")).read()
    declared = set(re.findall(r"^\s*(?:int|size_t|long long)\s+(mz_\w+)\s*\(", header, flags=re.M))
    assert declared == set(_cabi.EXPORTS), declared ^ set(_cabi.EXPORTS)
    lib = _cabi.load_library()
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.mz_version() >= 100


def test_struct_layout_matches_header():
    """ctypes mirrors must have the size the C compiler gives the header's structs."""
    import subprocess, tempfile
    from muzero_b200.kernels import _cabi
    src = '#include <stdio.h>\n#include "muzero_b200.h"\nint main(){printf("%zu %zu\\n", sizeof(mz_kv_store), sizeof(mz_decode_args));return 0;}\n'
    with tempfile.TemporaryDirectory() as td:
        c = os.path.join(td, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(td, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        a, b = map(int, subprocess.check_output([exe]).split())
    assert ctypes.sizeof(_cabi.KVStore) == a
    assert ctypes.sizeof(_cabi.DecodeArgs) == b


def test_argument_errors_are_reported_without_a_gpu():
    from muzero_b200.kernels import _cabi
    lib = _cabi.load_library()
    assert lib.mz_quantize_rows(None, 2, 4, 64, 9, 2.0, 1e-8, None, None, None, 1, None) == 1
    assert "bits" in _cabi.last_error()
    s = _cabi.KVStore()
    assert lib.mz_flush_kv(ctypes.byref(s), 64, 1e-8, None) == 1
    a = _cabi.DecodeArgs()
    assert lib.mz_decode_workspace_bytes(ctypes.byref(a)) == 0
    # the fused step validates before it launches anything, too
    assert lib.mz_decode_step_workspace_bytes(ctypes.byref(a), 128, 64) == 0
    assert lib.mz_decode_step(None, None, None, 0, 0, 128, 64, 0, 0, 1e-8, None) == 1
    a.store.group = 64
    assert lib.mz_decode_step(ctypes.byref(a), None, None, 0, 0, 128, 96, 0, 0, 1e-8, None) == 1
    assert "flush_unit" in _cabi.last_error()
    assert lib.mz_decode_step(ctypes.byref(a), None, None, 0, 0, 128, 64, 0, 0, 1e-8, None) == 4     # window has no room
    assert "window" in _cabi.last_error()


def test_cpu_tensors_are_rejected_not_silently_handled():
    import muzero_b200 as mz
    from muzero_b200.kernels import MuZeroKernelError
    with pytest.raises(MuZeroKernelError):
        mz.quantize_rows(torch.randn(4, 64), 4, 2.0, 1e-8, torch.float16)
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig())
    k = torch.randn(1, 2, 512, 64, dtype=torch.float16)
    with pytest.raises(MuZeroKernelError):
        layer.update(k, k.clone())


def test_config_matches_reference_contract():
    import muzero_b200 as mz
    cfg = mz.MuZeroConfig()
    assert (cfg.bits, cfg.q_group_size, cfg.residual_length, cfg.amax_dtype, cfg.decode_flush_by_group) == (4, 64, 128, "float16", True)
    assert mz.MuZeroConfig.from_dict({"bits": 2, "q_group_size": 32, "residual_length": 64, "junk": 1}).bits == 2
    for bad in (dict(bits=5), dict(bits=6), dict(amax_dtype="float8"), dict(backend="metal"), dict(q_group_size=0),
                dict(residual_length=100)):
        with pytest.raises(ValueError):
            mz.MuZeroConfig(**bad)
    mz.MuZeroConfig(residual_length=100, decode_flush_by_group=False)
    for bits in (1, 2, 3, 4, 7, 8):
        mz.MuZeroConfig(bits=bits)


def test_flush_policy():
    from muzero_b200.cache.policy import plan_flush, residual_capacity, grown_capacity
    kw = dict(residual_length=128, group=64, flush_by_group=True, logq_layout=False)
    assert plan_flush(key_len=4096, value_len=4096, decode_flush=False, **kw).key_tokens == 3968
    assert plan_flush(key_len=300, value_len=300, decode_flush=False, **kw).key_tokens == 128
    assert plan_flush(key_len=191, value_len=191, decode_flush=True, **kw).key_tokens == 0
    assert plan_flush(key_len=192, value_len=192, decode_flush=True, **kw) .key_tokens == 64
    kw4 = dict(residual_length=128, group=64, flush_by_group=False, logq_layout=False)
    assert plan_flush(key_len=192, value_len=192, decode_flush=True, **kw4).key_tokens == 0
    assert plan_flush(key_len=384, value_len=384, decode_flush=True, **kw4).key_tokens == 256
    assert plan_flush(key_len=192, value_len=192, decode_flush=False, **kw4).key_tokens == 64
    lq = plan_flush(key_len=200, value_len=200, residual_length=128, group=64, decode_flush=True, flush_by_group=False,
                    logq_layout=True)
    assert (lq.key_tokens, lq.value_tokens) == (64, 72)
    assert plan_flush(key_len=64, value_len=64, decode_flush=True, residual_length=0, group=64, flush_by_group=True,
                      logq_layout=False).key_tokens == 64
    cap = residual_capacity(129, 128, 64)
    assert cap % 256 == 0 and cap >= 128 + 2 * 256
    assert grown_capacity(0, 62) == 70 and grown_capacity(70, 71) >= 78 and grown_capacity(100, 50) == 100


def test_select_alpha_host_matches_reference(oracle, golden):
    import muzero_b200 as mz
    from muzero_b200.quantizer import select_alpha_key_block
    from muzero_b200.cache.layer import _select_alpha_value_block
    k, v, _ = oracle.synth_kv(2, 4, 1024, 128, 8, seed=7)
    a = golden.alpha
    for group in (32, 64, 128):
        kr, vr = oracle.key_rows(k, group), oracle.value_rows(v, group)
        for bits in (1, 2, 3, 4, 7, 8):
            assert mz.select_alpha(kr, bits=bits, q_group_size=group, kind="key") == a[f"key_rows_b{bits}_g{group}"]
            assert mz.select_alpha(vr, bits=bits, q_group_size=group, kind="value") == a[f"value_rows_b{bits}_g{group}"]
            assert mz.select_alpha(k, bits=bits, q_group_size=group, kind="key") == a[f"key_4d_b{bits}_g{group}"]
            assert mz.select_alpha(v, bits=bits, q_group_size=group, kind="value") == a[f"value_4d_b{bits}_g{group}"]
            # layout-aware variants used by the cache layer (no transposed copy), also on strided views
            kt = k.transpose(1, 2).contiguous().transpose(1, 2)
            assert select_alpha_key_block(kt, bits=bits, q_group_size=group) == a[f"key_rows_b{bits}_g{group}"]
            assert _select_alpha_value_block(v, bits=bits, group=group, d_pad=128, max_points=65536) == a[f"value_rows_b{bits}_g{group}"]
    heavy = torch.randn(4096, 64, generator=torch.Generator().manual_seed(3)) ** 3
    for bits in (1, 3, 8):
        assert mz.select_alpha(heavy, bits=bits, q_group_size=64, kind="key") == a[f"heavy_key_b{bits}"]
        assert mz.select_alpha(heavy, bits=bits, q_group_size=64, kind="value") == a[f"heavy_value_b{bits}"]


def test_patch_transformers_registers_and_is_idempotent():
    import muzero
    muzero.patch_transformers()
    muzero.patch_transformers()
    from transformers.cache_utils import CACHE_CLASS_REGISTRY
    for bits in (1, 2, 3, 4, 7, 8):
        assert f"mu_zero_{bits}bit" in CACHE_CLASS_REGISTRY
    cache = CACHE_CLASS_REGISTRY["mu_zero_4bit"](q_group_size=64, residual_length=128, quant_backend="cuda")
    assert isinstance(cache, muzero.MuZeroCache) and cache.cfg.bits == 4 and cache.cfg.backend == "cuda"
    import transformers.generation.configuration_utils as gcu
    assert "mu_zero_2bit" in gcu.ALL_CACHE_IMPLEMENTATIONS


def test_expand_table_host_equals_oracle(oracle):
    from muzero_b200.kernels.loader import expand_table_host
    for bits in (1, 4, 8):
        assert torch.equal(expand_table_host(bits, 2.0), oracle.expand_table_oracle(bits, 2.0))


def test_tile_partition_matches_bruteforce(tmp_path):
    """The decode kernel and its merge kernel find each warp's tiles with the same 32-bit functions
    (muzero_b200/csrc/mz_decode.cuh); they must agree with plain 64-bit arithmetic and tile the list."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    exe = tmp_path / "partition_check"
    src = os.path.join(os.path.dirname(__file__), "partition_check.cu")
    subprocess.run([nvcc, "-std=c++17", "-o", str(exe), src], check=True, capture_output=True)
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout
    assert "BAD" not in run.stdout and run.stdout.count(": ok") == 12


def test_prefill_deferral_rules(monkeypatch):
    """Which prompt blocks stay dense until the first decode step (host logic only).  Reference:
    muzero/integrations/transformers_patch.py:546-555 defers every block under generate();
    benchmarks/bench_throughput.py:244-279 quantizes chunk by chunk when it prefills in chunks."""
    import muzero_b200 as mz
    from muzero_b200.integrations.transformers_patch import MuZeroCache
    cfg = mz.MuZeroConfig(bits=4, q_group_size=64, residual_length=128)
    monkeypatch.delenv("MUZERO_QUANTIZE_PREFILL_CHUNKS", raising=False)
    cache = MuZeroCache(cfg)
    assert cache.prefill_block_defers(0) is False            # no deferral asked for
    cache.defer_prefill_quantization = True
    cache.single_shot_prefill = True
    assert cache.prefill_block_defers(0) is False            # the whole prompt in one block: quantized in its own update
    cache.single_shot_prefill = False
    assert cache.prefill_block_defers(0) is True             # chunked prefill keeps the reference's deferral ...
    monkeypatch.setenv("MUZERO_QUANTIZE_PREFILL_CHUNKS", "1")
    chunked = MuZeroCache(cfg)
    chunked.defer_prefill_quantization = True
    chunked.single_shot_prefill = False
    assert chunked.prefill_block_defers(0) is False          # ... unless chunks are to be quantized as they arrive
