"""GPU: the checked build of the library (compiled with -DMZ_BOUNDS).

Guarded global stores compare their index with the extent the host passed; an access outside it is skipped
and counted, never trapped, so the CUDA context stays usable.  The checked library is a second shared
object, selected through MUZERO_B200_LIB, so it is exercised in a child process: small shapes through the
cache layer (prefill flush, decode steps with every decode-attention kernel, a batch gather) must leave the
violation count at zero and still agree with the CPU oracle; a flush into a store that is declared full must
be counted and must leave the store untouched.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED_LIB = os.path.join(ROOT, "muzero_b200", "lib", "libmuzero_b200_bounds.so")

CHILD = r"""
import ctypes, sys, torch
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
from conftest import load_oracle
import muzero_b200 as mz
from muzero_b200.cache.attention import decode_attention
from muzero_b200.kernels._cabi import check, load_library, stream_ptr
lib = load_library()
orc = load_oracle()

def violations(reset=0):
    i, n, site = ctypes.c_longlong(), ctypes.c_longlong(), ctypes.c_int()
    c = lib.mz_bounds_violations(ctypes.byref(i), ctypes.byref(n), ctypes.byref(site), reset)
    return c, i.value, n.value, site.value

assert violations()[0] == 0, "not a checked build, or a dirty record: %r" % (violations(),)
for bits, gqa in ((4, 4), (2, 2), (3, 1)):
    KVH = 2
    k, v, q = orc.synth_kv(3, KVH, 64 * 7 + 50, 128, KVH * gqa, seed=900 + bits)
    cfg = mz.MuZeroConfig(bits=4, q_group_size=64, residual_length=128)
    cfg.bits = bits
    layer = mz.MuZeroCacheLayer(cfg)
    layer.update(k.cuda(), v.cuda(), {{"materialize_full_kv": False}})
    ref = orc.OracleCacheLayer(bits=bits, group=64, residual=128)
    ref.append(k, v)
    want = orc.decode_attention_oracle(q, ref, 0.088, gqa, compute_dtype=torch.float32)
    for which in (1, 2, 3, 4):                      # generic, SIMT tiles, mma.sync, tcgen05 (where they apply)
        prev = lib.mz_debug_force_kernel(which)
        try:
            got = decode_attention(layer, q.cuda(), 0.088, out_dtype=torch.float32)
        finally:
            lib.mz_debug_force_kernel(prev)
        err = (got.cpu() - want).abs().max().item()
        assert err <= 2e-3, (bits, gqa, which, err)
    # decode steps across a flush, then a batch gather
    for step in range(70):
        kn, vn, _ = orc.synth_kv(3, KVH, 1, 128, KVH * gqa, seed=5000 + step)
        layer.update(kn.cuda(), vn.cuda(), {{"materialize_full_kv": False}})
    layer.batch_select_indices(torch.tensor([2, 0], device="cuda"))
    c = violations()
    assert c[0] == 0, (bits, c)

# a store declared full: the flush must skip every store, count them, and change nothing
k, v, q = orc.synth_kv(2, 2, 64 * 4 + 128, 128, 8, seed=77)
layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=4, q_group_size=64, residual_length=128))
layer.update(k.cuda(), v.cuda(), {{"materialize_full_kv": False}})
assert layer.keys.shape[2] >= 64
s = layer._store_struct()
bufs = layer._bufs
before = {{n: t.clone() for n, t in bufs.items()}}
s.k_groups = bufs["pk"].shape[2]                   # no room left in either store
s.v_tokens = bufs["pv"].shape[2]
check(lib.mz_flush_kv(ctypes.byref(s), 64, 1e-8, stream_ptr(torch.device("cuda"))), "mz_flush_kv")
count, index, extent, site = violations(reset=1)
assert count > 0 and index >= extent and 1 <= site <= 6, (count, index, extent, site)
for n, t in bufs.items():                         # bit patterns: unused capacity is uninitialised and may hold NaN
    assert torch.equal(t.view(torch.uint8), before[n].view(torch.uint8)), n
assert violations()[0] == 0                        # cleared
torch.cuda.synchronize()
print("CHECKED-BUILD-OK", count, site)
"""


def test_checked_build_small_shapes():
    if not os.path.exists(CHECKED_LIB):
        pytest.skip("checked library not built (python -m muzero_b200.build --bounds)")
    env = dict(os.environ, MUZERO_B200_LIB=CHECKED_LIB)
    res = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT)], env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0 and "CHECKED-BUILD-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
