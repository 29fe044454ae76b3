"""GPU: the allocation-free decode entry point (``mz_decode_attention_static``).

Some users of this library cannot allocate device memory when they call it - a serving
process that handed its whole memory pool out at start-up, a latency-critical decode loop that
forbids cudaMalloc because it synchronises the device, a plug-in inside a runtime that owns the
allocator.  For them the library keeps the scratch of
the decode attention in a static 8 MiB device array.  This test drives the entry point through
the C ABI, twice in a row on different inputs (the array is shared and keeps old contents),
and checks each result against the ordinary entry point (same kernels, so the tolerance the
other attention tests use, 2e-3, is met with room to spare) and against the CPU oracle (the
reference's attention evaluated in fp32, same tolerance).  It lives in a file that pytest
collects last, so that a run that stops at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

from conftest import load_oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _layer(orc, seed, bits, batch, seq):
    import muzero_b200 as mz
    k, v, q = orc.synth_kv(batch, 2, seq, 128, 8, seed=seed)
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=bits, q_group_size=64, residual_length=128))
    layer.update(k.cuda(), v.cuda(), {"materialize_full_kv": False})
    ref = orc.OracleCacheLayer(bits=bits, group=64, residual=128)
    ref.append(k, v)
    layer.oracle_output = orc.decode_attention_oracle(q, ref, 0.088, 4, compute_dtype=torch.float32)
    return layer, q.cuda()


def _call(fn_name, layer, q, scaling):
    from muzero_b200.cache.attention import build_decode_args
    from muzero_b200.kernels._cabi import check, load_library, stream_ptr
    out = torch.empty(q.shape[0], 1, q.shape[1], 128, dtype=torch.float32, device=q.device)
    args = build_decode_args(layer, q, scaling, None, out)
    if fn_name == "mz_decode_attention_static":
        args.workspace, args.workspace_bytes = None, 0      # the static variant must not need them
    check(getattr(load_library(), fn_name)(ctypes.byref(args), stream_ptr(q.device)), fn_name)
    torch.cuda.synchronize()
    return out


def test_static_scratch_matches_workspace_variant_twice():
    orc = load_oracle()
    cases = [_layer(orc, 101, 4, 3, 700), _layer(orc, 202, 2, 2, 1300)]
    for layer, q in cases:                       # two calls in a row on the shared array
        want = _call("mz_decode_attention", layer, q, 0.088)
        got = _call("mz_decode_attention_static", layer, q, 0.088)
        assert torch.isfinite(got).all()
        assert (got - want).abs().max().item() <= TOL
        assert (got.cpu() - layer.oracle_output).abs().max().item() <= TOL
    # and once more on the first case, after the array was reused by the second
    layer, q = cases[0]
    again = _call("mz_decode_attention_static", layer, q, 0.088)
    assert (again - _call("mz_decode_attention", layer, q, 0.088)).abs().max().item() <= TOL
    assert (again.cpu() - layer.oracle_output).abs().max().item() <= TOL


def test_static_scratch_rejects_what_it_cannot_serve():
    from muzero_b200.cache.attention import build_decode_args
    from muzero_b200.kernels._cabi import last_error, load_library, stream_ptr
    orc = load_oracle()
    lib = load_library()
    layer, q = _layer(orc, 303, 4, 2, 700)
    out = torch.empty(2, 1, 8, 128, dtype=torch.float32, device="cuda")
    args = build_decode_args(layer, q, 0.088, None, out, splits=4096)     # 2*2 pairs * 4096 splits * 4 heads * 130 floats > 8 MiB
    assert lib.mz_decode_attention_static(ctypes.byref(args), stream_ptr(q.device)) == 4
    assert "static array holds" in last_error()
    import muzero_b200 as mz
    k, v, q64 = orc.synth_kv(1, 2, 300, 64, 4, seed=9)                     # head_dim 64 -> shape-generic kernel
    small = mz.MuZeroCacheLayer(mz.MuZeroConfig(residual_length=64))
    small.update(k.cuda(), v.cuda(), {"materialize_full_kv": False})
    out64 = torch.empty(1, 1, 4, 64, dtype=torch.float32, device="cuda")
    args = build_decode_args(small, q64.cuda(), 0.125, None, out64)
    assert lib.mz_decode_attention_static(ctypes.byref(args), stream_ptr(q.device)) == 2
    assert "shape-generic" in last_error()
