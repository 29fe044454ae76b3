"""GPU: MuZeroCacheLayer (flush, append, store layout, dequantization) against golden states and the oracle layer."""
import numpy as np
import pytest
import torch

from conftest import bits16, sha
from test_oracle_golden import build_case

pytestmark = pytest.mark.gpu
CASES = ["c4g64", "c2g64", "c3g32", "c8g128", "c1g64", "c7g64", "c4g64_d64", "c4g64_dec", "c2g64_dec4g",
         "c4g64_bf16meta", "c4g64_f32meta"]


def _meta_arr(t):
    t = t.detach().cpu().contiguous()
    return t.numpy() if t.dtype == torch.float32 else bits16(t)


def gpu_layer_from_meta(oracle, meta, hf_strides=False):
    import muzero_b200 as mz
    extra = dict(meta["extra"])
    cfg = mz.MuZeroConfig(bits=meta["bits"], q_group_size=meta["group"], residual_length=meta["residual"], **extra)
    layer = mz.MuZeroCacheLayer(cfg)
    k, v, q = oracle.synth_kv(meta["B"], meta["KVH"], meta["S"] + meta["steps"], meta["D"], meta["H"], seed=meta["seed"])
    S = meta["S"]
    kc, vc = k[:, :, :S].cuda(), v[:, :, :S].cuda()
    if hf_strides:   # the layout a model hands over: [B,S,KVH,D] transposed to [B,KVH,S,D]
        kc = kc.transpose(1, 2).contiguous().transpose(1, 2)
        vc = vc.transpose(1, 2).contiguous().transpose(1, 2)
    else:
        kc, vc = kc.contiguous(), vc.contiguous()
    layer.update(kc, vc, {"materialize_full_kv": False})
    for i in range(meta["steps"]):
        layer.update(k[:, :, S + i:S + i + 1].cuda(), v[:, :, S + i:S + i + 1].cuda(), {"materialize_full_kv": False})
    return layer, q.cuda()


@pytest.mark.parametrize("hf_strides", [False, True])
@pytest.mark.parametrize("name", CASES)
def test_layer_state_matches_reference(oracle, golden, name, hf_strides):
    meta = golden.layer_meta[name]
    layer, _ = gpu_layer_from_meta(oracle, meta, hf_strides)
    g = golden.layer
    assert np.array_equal(layer._packed_key_q.cpu().numpy(), g[name + "/packed_k"])
    assert np.array_equal(layer._packed_value_q.cpu().numpy(), g[name + "/packed_v"])
    for attr, nm in (("_key_mn", "k_mn"), ("_key_scale", "k_scale"), ("_value_mn", "v_mn"), ("_value_scale", "v_scale")):
        assert np.array_equal(_meta_arr(getattr(layer, attr)), g[f"{name}/{nm}"]), nm
    assert np.array_equal(bits16(layer.keys), g[name + "/res_k"])
    assert np.array_equal(bits16(layer.values), g[name + "/res_v"])
    assert [layer._selected_alpha_key, layer._selected_alpha_value] == list(g[name + "/alpha"])
    assert sha(layer._dequantize_key_prefix()) == meta["deq_bf16_sha"]["k"]
    assert sha(layer._dequantize_value_prefix()) == meta["deq_bf16_sha"]["v"]
    state = layer.get_attention_state()
    assert state["key_prefix_length"] == g[name + "/packed_k"].shape[2] * meta["group"] == state["value_prefix_length"]


def test_step_by_step_against_oracle_layer(oracle):
    """Prefill + 200 single-token updates: store, residual and lengths equal the oracle's after every step."""
    import muzero_b200 as mz
    k, v, _ = oracle.synth_kv(2, 2, 150 + 200, 128, 4, seed=21)
    ref = oracle.OracleCacheLayer(bits=4, group=32, residual=64)
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=4, q_group_size=32, residual_length=64))
    ref.append(k[:, :, :150].contiguous(), v[:, :, :150].contiguous())
    layer.update(k[:, :, :150].cuda().contiguous(), v[:, :, :150].cuda().contiguous(), {"materialize_full_kv": False})
    for i in range(150, 350):
        ref.append(k[:, :, i:i + 1].contiguous(), v[:, :, i:i + 1].contiguous())
        rk, rv = layer.update(k[:, :, i:i + 1].cuda(), v[:, :, i:i + 1].cuda(), {"materialize_full_kv": False})
        assert rk.shape[2] == ref.keys.shape[2] and layer.get_seq_length() == i + 1
        if i % 16 == 0 or i == 349:
            assert torch.equal(layer._packed_key_q.cpu(), ref.packed_k)
            assert torch.equal(layer._packed_value_q.cpu(), ref.packed_v)
            assert np.array_equal(bits16(layer._key_scale), bits16(ref.k_scale))
            assert np.array_equal(bits16(layer.keys), bits16(ref.keys))
            assert np.array_equal(bits16(layer.values), bits16(ref.values))


def test_range_dequant_and_full_materialisation(oracle):
    import muzero_b200 as mz
    k, v, _ = oracle.synth_kv(1, 2, 512, 128, 4, seed=33)
    ref = oracle.OracleCacheLayer(bits=4, group=64, residual=128)
    ref.append(k, v)
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig())
    layer.update(k.cuda(), v.cuda())
    kp, vp = ref.key_prefix(torch.bfloat16), ref.value_prefix(torch.bfloat16)
    assert np.array_equal(bits16(layer._dequantize_key_range(1, 4)), bits16(kp[:, :, 64:256].contiguous()))
    assert np.array_equal(bits16(layer._dequantize_value_range(100, 300)), bits16(vp[:, :, 100:300].contiguous()))
    k1, v1, _ = oracle.synth_kv(1, 2, 1, 128, 4, seed=34)
    fk, fv = layer.update(k1.cuda(), v1.cuda())       # default: full dense K/V
    assert fk.shape[2] == 513
    want = torch.cat([kp, ref.keys, k1], dim=2)
    assert np.array_equal(bits16(fk), bits16(want))


def test_reference_cache_suite():
    """The reference's own unit tests for the layer (tests/test_cache.py), on the CUDA path."""
    import muzero_b200 as mz

    def make(**kw):
        base = dict(bits=4, q_group_size=64, residual_length=128)
        base.update(kw)
        return mz.MuZeroCacheLayer(mz.MuZeroConfig(**base))

    def kv(bs, nh, sl, hd):
        return (torch.randn(bs, nh, sl, hd, device="cuda", dtype=torch.float16),
                torch.randn(bs, nh, sl, hd, device="cuda", dtype=torch.float16))

    layer = make()
    k, v = kv(1, 8, 512, 128)
    rk, rv = layer.update(k, v, {"materialize_full_kv": True})
    assert rk.shape == k.shape and rv.shape == v.shape
    assert layer._packed_key_q is not None and layer._packed_value_q is not None
    small = make()
    small.update(*kv(1, 8, 64, 128))
    assert small._packed_key_q is None
    k2, v2 = kv(1, 8, 1, 128)
    assert layer.update(k2, v2)[0].shape[-2] == 513 and layer.get_seq_length() == 513
    assert layer.update(*kv(1, 8, 1, 128), {"materialize_full_kv": False})[0].shape[-2] <= 129 + 64
    by_group = make(decode_flush_by_group=True)
    by_group.update(*kv(1, 8, 128, 128))
    assert by_group._packed_key_q is None
    for _ in range(64):
        by_group.update(*kv(1, 8, 1, 128), {"materialize_full_kv": False})
    assert by_group._packed_key_q.shape[2] == 1 and by_group._packed_value_q.shape[2] == 64
    assert by_group.keys.shape[2] == 128 and by_group.values.shape[2] == 128
    layer.reset()
    assert not layer.is_initialized and layer._packed_key_q is None and layer.cumulative_length == 0
    for bits in (2, 4, 8):
        l2 = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=bits, q_group_size=64, residual_length=64))
        k, v = kv(1, 4, 256, 64)
        assert l2.update(k, v, {"materialize_full_kv": True})[0].shape == k.shape


def test_crop_reorder_offload(oracle):
    import muzero_b200 as mz
    k, v, _ = oracle.synth_kv(3, 2, 400, 128, 4, seed=5)
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig())
    layer.update(k.cuda(), v.cuda())
    full_k, _ = layer._full_kv()
    layer.batch_select_indices(torch.tensor([2, 0], device="cuda"))
    sel_k, _ = layer._full_kv()
    assert torch.equal(sel_k, full_k[[2, 0]])
    layer.offload()
    assert not layer.keys.is_cuda and layer._packed_key_q.is_pinned()
    layer.prefetch()
    assert torch.equal(layer._full_kv()[0], full_k[[2, 0]])
    # beam-search style reorder with a repeated entry, then a repeat-interleave; decoding goes on afterwards
    layer.reorder_cache(torch.tensor([1, 1, 0], device="cuda"))
    assert torch.equal(layer._full_kv()[0], full_k[[0, 0, 2]])
    layer.batch_repeat_interleave(2)
    want = full_k[[0, 0, 0, 0, 2, 2]]
    assert torch.equal(layer._full_kv()[0], want) and layer.keys.shape[0] == 6
    layer.update(k[[0, 0, 0, 0, 2, 2], :, :1].cuda(), v[[0, 0, 0, 0, 2, 2], :, :1].cuda(), {"materialize_full_kv": False})
    assert layer.get_seq_length() == 401 and torch.equal(layer._full_kv()[0][:, :, :400], want)
    with pytest.raises(Exception):
        layer.batch_select_indices(torch.tensor([7], device="cuda"))
    layer.crop(100)
    assert layer.get_seq_length() == 100 and torch.equal(layer.keys, want[:, :, :100])


def test_batch_select_with_empty_residual_window(oracle):
    """residual_length=0: right after a flush the window holds no token; reindexing the batch must still
    carry it along, and decoding must go on with the new batch."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    k, v, q = oracle.synth_kv(3, 2, 257, 128, 8, seed=8)
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(residual_length=0))
    layer.update(k[:, :, :256].cuda().contiguous(), v[:, :, :256].cuda().contiguous(), {"materialize_full_kv": False})
    assert layer.keys.shape[2] == 0 and layer._key_group_count == 4
    layer.batch_select_indices(torch.tensor([2, 0], device="cuda"))
    assert layer.keys.shape[0] == 2 and layer._packed_key_q.shape[0] == 2
    layer.update(k[[2, 0], :, 256:257].cuda(), v[[2, 0], :, 256:257].cuda(), {"materialize_full_kv": False})
    ref = oracle.OracleCacheLayer(bits=4, group=64, residual=0)
    ref.append(k[[2, 0], :, :256].contiguous(), v[[2, 0], :, :256].contiguous())
    ref.append(k[[2, 0], :, 256:257].contiguous(), v[[2, 0], :, 256:257].contiguous())
    want = oracle.decode_attention_oracle(q[[2, 0]], ref, 0.09, 4, compute_dtype=torch.float32)
    got = decode_attention(layer, q[[2, 0]].cuda(), 0.09, out_dtype=torch.float32)
    assert (got.cpu() - want).abs().max().item() <= 2e-3


def test_first_block_with_unlike_key_value_strides(oracle):
    """B=1, KVH=1: size-1 dimensions make strides ambiguous, so the keys (fresh from RoPE, contiguous) and the
    values (a transposed view) of the first block can disagree in layout; the block is then copied."""
    import muzero_b200 as mz
    k, v, _ = oracle.synth_kv(1, 1, 300, 128, 4, seed=12)
    kc = k.cuda().contiguous()
    vc = v.cuda().transpose(1, 2).contiguous().transpose(1, 2)
    if vc.stride() == kc.stride():      # make the two layouts differ for sure: a batch stride no other size-1 view has
        vc = vc.as_strided(vc.shape, (vc.stride(0) * 3, vc.stride(1), vc.stride(2), 1))
    assert vc.stride() != kc.stride()
    want = mz.MuZeroCacheLayer(mz.MuZeroConfig())
    want.update(kc, v.cuda().contiguous(), {"materialize_full_kv": False})
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig())
    layer.update(kc, vc, {"materialize_full_kv": False})
    assert torch.equal(layer._packed_value_q, want._packed_value_q) and torch.equal(layer._packed_key_q, want._packed_key_q)
    assert torch.equal(layer.values, want.values) and torch.equal(layer.keys, want.keys)


@pytest.mark.gpu
@pytest.mark.parametrize("by_group,bits", [(True, 4), (False, 4), (True, 2)])
def test_decode_step_equals_update_then_attention(oracle, by_group, bits):
    """`MuZeroCacheLayer.decode_step` (one C call: append, flush when due, attention) against the two-call
    route over 600 steps: same outputs bit for bit, same store, same residual window, across flushes,
    store growth and the window sliding back to the front of its buffer."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    steps = 600
    k, v, _ = oracle.synth_kv(2, 2, 300 + steps, 128, 8, seed=11 + bits)
    gen = torch.Generator().manual_seed(5)
    qs = torch.randn(steps, 2, 8, 1, 128, generator=gen).to(torch.bfloat16).cuda()
    k, v = k.cuda(), v.cuda()
    cfg = dict(bits=bits, q_group_size=64, residual_length=128, decode_flush_by_group=by_group)
    a, b = mz.MuZeroCacheLayer(mz.MuZeroConfig(**cfg)), mz.MuZeroCacheLayer(mz.MuZeroConfig(**cfg))
    for layer in (a, b):
        layer.update(k[:, :, :300].contiguous(), v[:, :, :300].contiguous(), {"materialize_full_kv": False})
    ref = oracle.OracleCacheLayer(bits=bits, group=64, residual=128, flush_by_group=by_group)
    ref.append(k[:, :, :300].cpu().contiguous(), v[:, :, :300].cpu().contiguous())
    fast = 0
    for i in range(steps):
        kn, vn = k[:, :, 300 + i:301 + i], v[:, :, 300 + i:301 + i]
        a.update(kn, vn, {"materialize_full_kv": False})
        want = decode_attention(a, qs[i], 0.09)
        before = b._res_start
        got = b.decode_step(kn, vn, qs[i], 0.09)
        fast += int(b._res_start >= before)
        assert torch.equal(got, want), i
        ref.append(kn.cpu().contiguous(), vn.cpu().contiguous())
        if i % 97 == 0 or i == steps - 1:      # the one-call step against the CPU oracle, directly
            exact = oracle.decode_attention_oracle(qs[i].cpu(), ref, 0.09, 4, compute_dtype=torch.float32)
            err = (got.float().cpu() - exact).abs()
            assert bool((err <= 2e-3 + exact.abs() * 2.0 ** -8).all()), (i, err.max().item())
        assert (b._key_group_count, b._value_storage_len, b.keys.shape[2], b.cumulative_length) == \
               (a._key_group_count, a._value_storage_len, a.keys.shape[2], a.cumulative_length), i
    assert torch.equal(a._packed_key_q, b._packed_key_q) and torch.equal(a._packed_value_q, b._packed_value_q)
    assert torch.equal(a._key_mn, b._key_mn) and torch.equal(a._value_scale, b._value_scale)
    assert torch.equal(a.keys, b.keys) and torch.equal(a.values, b.values)
    assert a._key_group_count > 4 and fast > steps // 2


@pytest.mark.gpu
def test_decode_step_with_mask_and_refusals(oracle):
    """Additive mask covering the token of the step; a mask that is one token short is refused."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    from muzero_b200.kernels._cabi import MuZeroKernelError
    k, v, q = oracle.synth_kv(2, 2, 401, 128, 8, seed=3)
    k, v, q = k.cuda(), v.cuda(), q.cuda()
    a, b = mz.MuZeroCacheLayer(mz.MuZeroConfig()), mz.MuZeroCacheLayer(mz.MuZeroConfig())
    for layer in (a, b):
        layer.update(k[:, :, :399].contiguous(), v[:, :, :399].contiguous(), {"materialize_full_kv": False})
        layer.update(k[:, :, 399:400], v[:, :, 399:400], {"materialize_full_kv": False})    # window now lives in its buffer
    mask = torch.zeros(2, 1, 1, 401, device="cuda")
    mask[0, ..., :50] = -1e4
    mask[1, ..., 395:] = -2.0
    a.update(k[:, :, 400:401], v[:, :, 400:401], {"materialize_full_kv": False})
    want = decode_attention(a, q, 0.09, mask)
    got = b.decode_step(k[:, :, 400:401], v[:, :, 400:401], q, 0.09, mask)
    assert torch.equal(got, want)
    with pytest.raises(MuZeroKernelError):
        b.decode_step(k[:, :, 400:401], v[:, :, 400:401], q, 0.09, mask)      # 402 tokens now, mask has 401


@pytest.mark.parametrize("hf_strides", [False, True])
@pytest.mark.parametrize("name", ["c4g64_logq", "c4g64_logq_dec", "c2g32_logq_dec"])
def test_logq_layout_matches_reference(oracle, golden, name, hf_strides, monkeypatch):
    """`logq_compatible_layout=True`: keys flush by whole groups, values token by token, so the value
    prefix runs ahead; store, residual windows and attention against the reference's own run.  The
    attention goes through the fused kernel (the two-kernel route is for other head sizes only)."""
    from muzero_b200.cache import attention as attention_module
    from muzero_b200.cache.attention import decode_attention

    def not_here(*a, **kw):
        raise AssertionError("head_dim 128 must take the fused kernel")
    monkeypatch.setattr(attention_module, "_decode_attention_unaligned", not_here)
    meta, g = golden.layer_logq_meta[name], golden.layer_logq
    layer, q = gpu_layer_from_meta(oracle, meta, hf_strides)
    assert np.array_equal(layer._packed_key_q.cpu().numpy(), g[name + "/packed_k"])
    assert np.array_equal(layer._packed_value_q.cpu().numpy(), g[name + "/packed_v"])
    for attr, nm in (("_key_mn", "k_mn"), ("_key_scale", "k_scale"), ("_value_mn", "v_mn"), ("_value_scale", "v_scale")):
        assert np.array_equal(_meta_arr(getattr(layer, attr)), g[f"{name}/{nm}"]), nm
    assert np.array_equal(bits16(layer.keys), g[name + "/res_k"])
    assert np.array_equal(bits16(layer.values), g[name + "/res_v"])
    assert [layer._selected_alpha_key, layer._selected_alpha_value] == list(g[name + "/alpha"])
    assert sha(layer._dequantize_key_prefix()) == meta["deq_bf16_sha"]["k"]
    assert sha(layer._dequantize_value_prefix()) == meta["deq_bf16_sha"]["v"]
    state = layer.get_attention_state()
    assert state["value_prefix_length"] > state["key_prefix_length"] > 0
    ref = torch.from_numpy(g[name + "/attn_fp32"])
    out = decode_attention(layer, q, meta["D"] ** -0.5, out_dtype=torch.float32)
    assert (out.cpu() - ref).abs().max().item() <= 2e-3
    k_full, v_full = layer._full_kv()
    assert k_full.shape == v_full.shape and k_full.shape[2] == meta["S"] + meta["steps"]
