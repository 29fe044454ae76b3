"""GPU: fused decode attention through the C-ABI against the reference's fp32 evaluation
(golden) and the oracle.  Tolerance: max-abs 2e-3 on fp32 output; bf16 output adds half a
bf16 ulp of the value (the rounding of the output itself)."""
import numpy as np
import pytest
import torch

from conftest import bits16, from_bits16, sha
from test_gpu_layer import CASES, gpu_layer_from_meta

pytestmark = pytest.mark.gpu
TOL = 2e-3
# Two runs that cut the tiles into different per-warp ranges agree to the rounding of the tensor-core
# operands (probabilities become fp16 relative to the running maximum of a warp's range), not to fp32
# summation order; the same launch geometry repeats bit for bit.
SPLIT_TOL = 5e-4


def bf16_half_ulp(x: torch.Tensor) -> torch.Tensor:
    e = torch.floor(torch.log2(x.abs().clamp_min(1e-30)))
    return torch.pow(2.0, e - 8)


def check_output(out_f32, out_bf16, ref):
    assert out_f32.shape == ref.shape
    err = (out_f32.cpu() - ref).abs().max().item()
    assert err <= TOL, f"fp32 output max-abs error {err}"
    slack = TOL + bf16_half_ulp(ref)
    assert bool(((out_bf16.float().cpu() - ref).abs() <= slack).all())
    return err


@pytest.mark.parametrize("name", CASES)
def test_attention_golden_cases(oracle, golden, name):
    from muzero_b200.cache.attention import decode_attention
    meta = golden.layer_meta[name]
    layer, q = gpu_layer_from_meta(oracle, meta)
    ref = torch.from_numpy(golden.layer[name + "/attn_fp32"])
    scaling = meta["D"] ** -0.5
    o32 = decode_attention(layer, q, scaling, out_dtype=torch.float32)
    obf = decode_attention(layer, q, scaling)
    check_output(o32, obf, ref)
    # split count must not matter beyond fp32 summation order; results are deterministic
    for splits in (1, 2, 5, 64):
        o = decode_attention(layer, q, scaling, out_dtype=torch.float32, splits=splits)
        assert (o - o32).abs().max().item() < SPLIT_TOL
    again = decode_attention(layer, q, scaling, out_dtype=torch.float32)
    assert torch.equal(again, o32)


@pytest.mark.parametrize("bits", [4, 2])
def test_config0_full(oracle, golden, bits):
    """Batch 1 x 8 kv heads x 4096 tokens, 32 query heads, 4-bit, group 64, residual 128: codes/metadata bit-exact (sha256 of the reference's tensors), attention within 2e-3."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    k, v, q = oracle.synth_kv(1, 8, 4096, 128, 32, seed=0)
    m = golden.config0_meta[f"b{bits}"]
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=bits, q_group_size=64, residual_length=128))
    layer.update(k.cuda(), v.cuda(), {"materialize_full_kv": False})
    assert sha(layer._packed_key_q) == m["packed_k"] and sha(layer._packed_value_q) == m["packed_v"]
    assert sha(layer._key_mn) == m["k_mn"] and sha(layer._key_scale) == m["k_scale"]
    assert sha(layer._value_mn) == m["v_mn"] and sha(layer._value_scale) == m["v_scale"]
    assert sha(layer._dequantize_key_prefix()) == m["deq_k_bf16"]
    assert sha(layer._dequantize_value_prefix()) == m["deq_v_bf16"]
    ref = torch.from_numpy(golden.config0[f"b{bits}_attn_fp32"])
    o32 = decode_attention(layer, q.cuda(), 128 ** -0.5, out_dtype=torch.float32)
    obf = decode_attention(layer, q.cuda(), 128 ** -0.5)
    check_output(o32, obf, ref)


def _oracle_and_gpu_layers(oracle, B, KVH, H, S, D, bits, group, residual, seed, steps=0):
    import muzero_b200 as mz
    k, v, q = oracle.synth_kv(B, KVH, S + steps, D, H, seed=seed)
    ref = oracle.OracleCacheLayer(bits=bits, group=group, residual=residual)
    cfg = mz.MuZeroConfig(bits=4, q_group_size=group, residual_length=residual)
    cfg.bits = bits     # 5 and 6 bits are outside the config's list but inside the kernels' range
    layer = mz.MuZeroCacheLayer(cfg)
    ref.append(k[:, :, :S].contiguous(), v[:, :, :S].contiguous())
    layer.update(k[:, :, :S].cuda().contiguous(), v[:, :, :S].cuda().contiguous(), {"materialize_full_kv": False})
    for i in range(S, S + steps):
        ref.append(k[:, :, i:i + 1].contiguous(), v[:, :, i:i + 1].contiguous())
        layer.update(k[:, :, i:i + 1].cuda(), v[:, :, i:i + 1].cuda(), {"materialize_full_kv": False})
    return ref, layer, q


@pytest.mark.parametrize("bits,group", [(1, 32), (3, 128), (5, 32), (5, 128), (6, 64), (7, 32), (8, 128), (4, 32), (2, 128), (1, 128), (8, 32)])
def test_any_bits_and_groups_vs_oracle(oracle, bits, group):
    from muzero_b200.cache.attention import decode_attention
    ref, layer, q = _oracle_and_gpu_layers(oracle, 2, 2, 8, 700, 128, bits, group, 128, seed=bits * 10 + group, steps=3)
    want = oracle.decode_attention_oracle(q, ref, 128 ** -0.5, 4, compute_dtype=torch.float32)
    o32 = decode_attention(layer, q.cuda(), 128 ** -0.5, out_dtype=torch.float32)
    obf = decode_attention(layer, q.cuda(), 128 ** -0.5)
    check_output(o32, obf, want)


@pytest.mark.parametrize("gqa,D", [(1, 128), (2, 128), (8, 128), (4, 64), (4, 16), (3, 96)])
def test_head_shapes(oracle, gqa, D):
    from muzero_b200.cache.attention import decode_attention
    ref, layer, q = _oracle_and_gpu_layers(oracle, 2, 2, 2 * gqa, 333, D, 4, 64, 64, seed=gqa * 100 + D, steps=70)
    want = oracle.decode_attention_oracle(q, ref, D ** -0.5, gqa, compute_dtype=torch.float32)
    o32 = decode_attention(layer, q.cuda(), D ** -0.5, out_dtype=torch.float32)
    check_output(o32, decode_attention(layer, q.cuda(), D ** -0.5), want)


def test_residual_only_and_additive_mask(oracle):
    from muzero_b200.cache.attention import decode_attention
    ref, layer, q = _oracle_and_gpu_layers(oracle, 2, 2, 8, 100, 128, 4, 64, 128, seed=77)
    assert layer._packed_key_q is None
    want = oracle.decode_attention_oracle(q, ref, 0.1, 4, compute_dtype=torch.float32)
    check_output(decode_attention(layer, q.cuda(), 0.1, out_dtype=torch.float32), decode_attention(layer, q.cuda(), 0.1), want)
    ref, layer, q = _oracle_and_gpu_layers(oracle, 2, 2, 8, 500, 128, 4, 64, 128, seed=78, steps=5)
    total = 505
    mask = torch.zeros(2, 1, 1, total + 3)
    mask[0, ..., :37] = torch.finfo(torch.bfloat16).min      # left padding of sequence 0
    mask[1, ..., 400:450] = -5.0
    want = oracle.decode_attention_oracle(q, ref, 0.09, 4, mask=mask, compute_dtype=torch.float32)
    for mdt in (torch.float32, torch.bfloat16):
        got = decode_attention(layer, q.cuda(), 0.09, mask.to(mdt).cuda(), out_dtype=torch.float32)
        assert (got.cpu() - want).abs().max().item() <= TOL


def test_partials_merge_like_a_kv_split(oracle):
    """Two stores holding the two halves of one sequence: merged partial triples equal the one-store result."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention, decode_attention_partial, lse_merge
    k, v, q = oracle.synth_kv(2, 2, 1024, 128, 8, seed=91)
    whole = mz.MuZeroCacheLayer(mz.MuZeroConfig(residual_length=0))
    whole.update(k.cuda(), v.cuda(), {"materialize_full_kv": False})
    a = mz.MuZeroCacheLayer(mz.MuZeroConfig(residual_length=0))
    a.update(k[:, :, :512].cuda().contiguous(), v[:, :, :512].cuda().contiguous(), {"materialize_full_kv": False})
    b = mz.MuZeroCacheLayer(mz.MuZeroConfig(residual_length=0))
    b.update(k[:, :, 512:].cuda().contiguous(), v[:, :, 512:].cuda().contiguous(), {"materialize_full_kv": False})
    qc = q.cuda()
    pa, pb = decode_attention_partial(a, qc, 0.088), decode_attention_partial(b, qc, 0.088)
    merged = lse_merge(torch.stack([pa[0], pb[0]]), torch.stack([pa[1], pb[1]]), torch.stack([pa[2], pb[2]]), torch.float32)
    one = decode_attention(whole, qc, 0.088, out_dtype=torch.float32)
    assert (merged - one).abs().max().item() < SPLIT_TOL
    m, l, acc = (t.cpu() for t in pa)
    ora = oracle.OracleCacheLayer(bits=4, group=64, residual=0)
    ora.append(k[:, :, :512].contiguous(), v[:, :, :512].contiguous())
    om, ol, oacc = oracle.attention_partial_oracle(q, ora.key_prefix(torch.float32), ora.value_prefix(torch.float32), 0.088, 4)
    assert (m - om).abs().max().item() < 1e-4
    assert ((acc / l.unsqueeze(-1)) - (oacc / ol.unsqueeze(-1))).abs().max().item() < TOL


def test_two_kernel_api_qk_and_av(oracle):
    """mu_zero_qk_cuda / mu_zero_av_cuda with the reference's argument order."""
    from muzero_b200.kernels import mu_zero_qk_cuda, mu_zero_av_cuda
    ref, layer, q = _oracle_and_gpu_layers(oracle, 2, 2, 8, 448, 128, 4, 64, 64, seed=12)
    qc = q.cuda()
    S = layer._packed_key_q.shape[2] * 64
    logits = torch.empty(2, 8, S, dtype=torch.float32, device="cuda")
    mu_zero_qk_cuda(qc, layer._packed_key_q.contiguous(), layer._key_mn.contiguous(), layer._key_scale.contiguous(), logits,
                    4, 2.0, 4, 0.088)
    kd = ref.key_prefix(torch.float32).repeat_interleave(4, dim=1)
    want = torch.einsum("bhd,bhsd->bhs", q.float().squeeze(2), kd) * 0.088
    assert (logits.cpu() - want).abs().max().item() < 1e-3
    w = torch.softmax(want, dim=-1).cuda()
    out = torch.empty(2, 8, 128, dtype=torch.float32, device="cuda")
    mu_zero_av_cuda(w, layer._packed_value_q.contiguous(), layer._value_mn.contiguous(), layer._value_scale.contiguous(), out,
                    4, 2.0, 4, 64)
    vd = ref.value_prefix(torch.float32).repeat_interleave(4, dim=1)
    assert (out.cpu() - torch.einsum("bhs,bhsd->bhd", w.cpu(), vd)).abs().max().item() < 1e-4


def test_hook_contract_and_stats(oracle):
    from types import SimpleNamespace
    import muzero_b200 as mz
    ref, layer, q = _oracle_and_gpu_layers(oracle, 1, 2, 8, 300, 128, 4, 64, 128, seed=3)
    mz.reset_mu_zero_decode_stats()
    mod = SimpleNamespace(num_key_value_groups=4)
    out, w = mz.mu_zero_decode_attention_forward(mod, q.cuda(), None, 0.088, layer.get_attention_state())
    assert w is None and out.shape == (1, 1, 8, 128) and out.dtype == torch.bfloat16 and out.is_contiguous()
    assert mz.mu_zero_decode_attention_forward(mod, torch.cat([q, q], dim=2).cuda(), None, 0.088, layer.get_attention_state()) is None
    assert mz.mu_zero_decode_attention_forward(mod, q.cuda(), None, 0.088, {}) is None
    st = mz.get_mu_zero_decode_stats()
    assert st["calls"] == 1 and st["returns"] == 1 and st["fused_qk_success"] == 1 and st["fused_av_success"] == 1
    assert st["non_decode_query"] == 1 and st["missing_layer"] == 1


@pytest.mark.parametrize("dtype", [torch.float16])
def test_fp16_cache(oracle, dtype):
    """K/V, query and residual in fp16 (the reference's unit tests use fp16 caches)."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    k, v, q = oracle.synth_kv(2, 2, 450, 128, 8, seed=55, dtype=dtype)
    ref = oracle.OracleCacheLayer(bits=4, group=64, residual=128)
    ref.append(k, v)
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig())
    layer.update(k.cuda(), v.cuda(), {"materialize_full_kv": False})
    assert torch.equal(layer._packed_key_q.cpu(), ref.packed_k) and torch.equal(layer._packed_value_q.cpu(), ref.packed_v)
    want = oracle.decode_attention_oracle(q, ref, 128 ** -0.5, 4, compute_dtype=torch.float32)
    got = decode_attention(layer, q.cuda(), 128 ** -0.5, out_dtype=torch.float32)
    assert (got.cpu() - want).abs().max().item() <= TOL
    assert decode_attention(layer, q.cuda(), 128 ** -0.5).dtype == torch.float16


def test_edge_lengths(oracle):
    """One residual token only; residual_length 0 with everything flushed; ragged residual tile."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    for S, R, steps in ((1, 128, 0), (64, 0, 0), (64, 0, 1), (129, 128, 0), (191, 64, 2)):
        k, v, q = oracle.synth_kv(1, 2, S + steps, 128, 8, seed=S + R)
        ref = oracle.OracleCacheLayer(bits=4, group=64, residual=R)
        layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(residual_length=R))
        ref.append(k[:, :, :S].contiguous(), v[:, :, :S].contiguous())
        layer.update(k[:, :, :S].cuda().contiguous(), v[:, :, :S].cuda().contiguous(), {"materialize_full_kv": False})
        for i in range(S, S + steps):
            ref.append(k[:, :, i:i + 1].contiguous(), v[:, :, i:i + 1].contiguous())
            layer.update(k[:, :, i:i + 1].cuda(), v[:, :, i:i + 1].cuda(), {"materialize_full_kv": False})
        want = oracle.decode_attention_oracle(q, ref, 0.09, 4, compute_dtype=torch.float32)
        got = decode_attention(layer, q.cuda(), 0.09, out_dtype=torch.float32)
        assert (got.cpu() - want).abs().max().item() <= TOL, (S, R, steps)


def test_long_context_many_warps(oracle):
    """32k tokens of one sequence: every warp of the grid gets a slice of the same (b, kv head) pair."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    k, v, q = oracle.synth_kv(1, 1, 32768 + 100, 128, 4, seed=99)
    ref = oracle.OracleCacheLayer(bits=2, group=64, residual=128, alpha_key=2.0, alpha_value=2.0)
    ref.append(k, v)
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=2, alpha_key=2.0, alpha_value=2.0))
    layer.update(k.cuda(), v.cuda(), {"materialize_full_kv": False})
    assert torch.equal(layer._packed_key_q.cpu(), ref.packed_k)
    want = oracle.decode_attention_oracle(q, ref, 128 ** -0.5, 4, compute_dtype=torch.float32)
    got = decode_attention(layer, q.cuda(), 128 ** -0.5, out_dtype=torch.float32)
    assert (got.cpu() - want).abs().max().item() <= TOL


@pytest.mark.parametrize("bits,group,gqa", [(4, 128, 8), (4, 32, 4), (2, 128, 2), (3, 64, 1)])
def test_masks_over_residual_tiles_and_wide_groups(oracle, bits, group, gqa):
    """Additive mask reaching into packed tiles and into the ragged last residual tile, for tile shapes
    other than the headline one (two-pass codebooks at G=128, 8 heads per kv head, 1 head)."""
    from muzero_b200.cache.attention import decode_attention
    ref, layer, q = _oracle_and_gpu_layers(oracle, 3, 2, 2 * gqa, 700, 128, bits, group, 128, seed=bits + group + gqa, steps=5)
    total = 705
    mask = torch.zeros(3, 1, 1, total)
    mask[0, ..., :70] = torch.finfo(torch.bfloat16).min
    mask[1, ..., 560:650] = -4.0
    mask[2, ..., 690:] = torch.finfo(torch.bfloat16).min
    want = oracle.decode_attention_oracle(q, ref, 0.09, gqa, mask=mask, compute_dtype=torch.float32)
    got = decode_attention(layer, q.cuda(), 0.09, mask.cuda(), out_dtype=torch.float32)
    assert (got.cpu() - want).abs().max().item() <= TOL


def test_many_pairs_and_split_counts_beyond_16_bits(oracle):
    """24 (batch, kv head) pairs: warps cross pair boundaries inside packed and residual tiles.  Then a split
    count that makes more than 65535 warps (the 64-bit branch of the tile partition) must give the same result."""
    from muzero_b200.cache.attention import decode_attention
    ref, layer, q = _oracle_and_gpu_layers(oracle, 6, 4, 16, 700, 128, 4, 64, 128, seed=606, steps=2)
    want = oracle.decode_attention_oracle(q, ref, 0.09, 4, compute_dtype=torch.float32)
    got = decode_attention(layer, q.cuda(), 0.09, out_dtype=torch.float32)
    assert (got.cpu() - want).abs().max().item() <= TOL
    for splits in (3, 17, 3000):          # 24 * 3000 = 72,000 warps
        again = decode_attention(layer, q.cuda(), 0.09, out_dtype=torch.float32, splits=splits)
        assert (again - got).abs().max().item() < SPLIT_TOL, splits


@pytest.mark.parametrize("which,name", [(1, "generic"), (2, "tiles"), (3, "mma"), (4, "umma")])
def test_every_kernel_against_the_oracle(oracle, which, name):
    """The four decode kernels on the same caches (4- and 2-bit, group 64, a pair boundary inside a worker's range,
    an odd number of tiles, a mask): each within 2e-3 of the oracle.  `umma` is the tcgen05 / tensor-memory kernel,
    which the automatic selection does not use yet."""
    from muzero_b200.cache.attention import decode_attention
    from muzero_b200.kernels._cabi import load_library
    lib = load_library()
    before = lib.mz_debug_force_kernel(which)
    try:
        for bits, S, steps in ((4, 1000, 3), (2, 600, 70)):
            ref, layer, q = _oracle_and_gpu_layers(oracle, 3, 2, 8, S, 128, bits, 64, 128, seed=900 + bits, steps=steps)
            total = S + steps
            mask = torch.zeros(3, 1, 1, total)
            mask[1, ..., 100:260] = -3.0
            mask[2, ..., :33] = torch.finfo(torch.bfloat16).min
            for m in (None, mask):
                want = oracle.decode_attention_oracle(q, ref, 0.09, 4, mask=m, compute_dtype=torch.float32)
                got = decode_attention(layer, q.cuda(), 0.09, None if m is None else m.cuda(), out_dtype=torch.float32)
                err = (got.cpu() - want).abs().max().item()
                assert err <= TOL, (name, bits, m is not None, err)
    finally:
        lib.mz_debug_force_kernel(before)
