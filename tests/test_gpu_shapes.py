"""GPU: parity at the benchmarked and at the long-context shapes, where the launch geometry differs from the
small cases: warps that cross (batch, kv head) boundaries, two segments per warp, hundreds of pairs, and one
pair cut over every warp of the grid.

The CUDA results of the full launch are compared with the CPU oracle on a few sequences (or one (batch, kv
head) pair) sampled across the batch: packed codes and metadata bit for bit, attention within 2e-3 on the
fp32 output, the tolerance of the other attention tests."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _gpu_batch_with_known_rows(oracle, B, KVH, S, H, rows, seed):
    """A [B,KVH,S,128] K/V batch drawn on the device, with the sequences `rows` replaced by CPU-drawn ones
    (the oracle sees exactly those bits).  Returns device K, V, q and the CPU copies of the known rows."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    chan = torch.exp(torch.randn(128, device="cuda", generator=gen))
    k = (torch.randn(B, KVH, S, 128, device="cuda", generator=gen) * chan).to(torch.bfloat16)
    v = torch.randn(B, KVH, S, 128, device="cuda", generator=gen).to(torch.bfloat16)
    q = torch.randn(B, H, 1, 128, device="cuda", generator=gen).to(torch.bfloat16)
    kc, vc, qc = oracle.synth_kv(len(rows), KVH, S, 128, H, seed=seed + 1)
    idx = torch.tensor(rows, device="cuda")
    k[idx], v[idx], q[idx] = kc.cuda(), vc.cuda(), qc.cuda()
    return k, v, q, kc, vc, qc


@pytest.mark.parametrize("bits", [4, 2])
def test_benchmarked_shape_batch64(oracle, bits):
    """Batch 64 x 8 kv heads x (4096 packed + 128 residual) tokens, 32 query heads, group 64: the shape bench.py
    times.  Sequences 0, 21, 42 and 63 are checked against the oracle."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    rows = [0, 21, 42, 63]
    k, v, q, kc, vc, qc = _gpu_batch_with_known_rows(oracle, 64, 8, 4096 + 128, 32, rows, seed=640 + bits)
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=bits, q_group_size=64, residual_length=128, alpha_key=2.0, alpha_value=2.0))
    layer.update(k, v, {"materialize_full_kv": False})
    del k, v
    assert layer._key_group_count == 64 and layer.keys.shape[2] == 128
    got = decode_attention(layer, q, 128 ** -0.5, out_dtype=torch.float32)
    got_bf = decode_attention(layer, q, 128 ** -0.5)
    for i, r in enumerate(rows):
        ref = oracle.OracleCacheLayer(bits=bits, group=64, residual=128, alpha_key=2.0, alpha_value=2.0)
        ref.append(kc[i:i + 1], vc[i:i + 1])
        assert torch.equal(layer._packed_key_q[r:r + 1].cpu(), ref.packed_k), r
        assert torch.equal(layer._packed_value_q[r:r + 1].cpu(), ref.packed_v), r
        assert torch.equal(layer._key_mn[r:r + 1].cpu(), ref.k_mn) and torch.equal(layer._value_scale[r:r + 1].cpu(), ref.v_scale), r
        want = oracle.decode_attention_oracle(qc[i:i + 1], ref, 128 ** -0.5, 4, compute_dtype=torch.float32)
        err = (got[r:r + 1].cpu() - want).abs().max().item()
        assert err <= TOL, (r, err)
        half_ulp = torch.pow(2.0, torch.floor(torch.log2(want.abs().clamp_min(1e-30))) - 8)
        assert bool(((got_bf[r:r + 1].float().cpu() - want).abs() <= TOL + half_ulp).all()), r


@pytest.mark.parametrize("bits,group", [(1, 32), (3, 128), (5, 32), (8, 128), (4, 64), (2, 64)])
def test_long_context_131k(oracle, bits, group):
    """One context of 131,072 quantized tokens + 128 residual, batch 2 x 8 kv heads x 32 query heads (the shape of
    the KV-split workload on one GPU); the pair (batch 1, kv head 5) is checked against the oracle."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    B, KVH, H, S = 2, 8, 32, 131072 + 128
    b0, h0 = 1, 5
    gen = torch.Generator(device="cuda").manual_seed(1310 + bits + group)
    k = torch.randn(B, KVH, S, 128, device="cuda", generator=gen).to(torch.bfloat16)
    v = torch.randn(B, KVH, S, 128, device="cuda", generator=gen).to(torch.bfloat16)
    q = torch.randn(B, H, 1, 128, device="cuda", generator=gen).to(torch.bfloat16)
    kc, vc, qc = oracle.synth_kv(1, 1, S, 128, 4, seed=77 + bits)
    k[b0, h0], v[b0, h0], q[b0, 4 * h0:4 * h0 + 4] = kc[0, 0].cuda(), vc[0, 0].cuda(), qc[0].cuda()
    alpha_k = 4.0 if bits == 1 else 2.0          # what the reference's selection rule picks on this distribution
    cfg = mz.MuZeroConfig(bits=4, q_group_size=group, residual_length=128, alpha_key=alpha_k, alpha_value=2.0)
    cfg.bits = bits                              # 5 bits: outside the config's list, inside the kernels' range
    layer = mz.MuZeroCacheLayer(cfg)
    layer.update(k, v, {"materialize_full_kv": False})
    del k, v
    ref = oracle.OracleCacheLayer(bits=bits, group=group, residual=128, alpha_key=alpha_k, alpha_value=2.0)
    ref.append(kc, vc)
    assert torch.equal(layer._packed_key_q[b0:b0 + 1, h0:h0 + 1].cpu(), ref.packed_k)
    assert torch.equal(layer._packed_value_q[b0:b0 + 1, h0:h0 + 1].cpu(), ref.packed_v)
    want = oracle.decode_attention_oracle(qc, ref, 128 ** -0.5, 4, compute_dtype=torch.float32)
    got = decode_attention(layer, q, 128 ** -0.5, out_dtype=torch.float32)
    err = (got[b0:b0 + 1, :, 4 * h0:4 * h0 + 4].cpu() - want).abs().max().item()
    assert err <= TOL, err


@pytest.mark.parametrize("bits,gqa", [(4, 4), (2, 2)])
def test_split_launch_with_mask_and_ragged_window(oracle, bits, gqa):
    """Enough packed tiles to fill every warp of the machine twice (16 x 8 pairs x 32 groups), so that the
    tensor-core kernel splits its launch into CTAs for packed tiles and CTAs for residual tiles; a residual window
    of 150 tokens (a ragged last tile), a left-padding mask and a mask over packed and residual tokens.  Sequences
    0, 7 and 15 are checked against the oracle, as normalised output and as the merged (m, l, acc) triple."""
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention, decode_attention_partial_packed
    B, KVH, S = 16, 8, 2048 + 150
    H = KVH * gqa
    rows = [0, 7, 15]
    k, v, q, kc, vc, qc = _gpu_batch_with_known_rows(oracle, B, KVH, S, H, rows, seed=2200 + bits)
    layer = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=bits, q_group_size=64, residual_length=128, alpha_key=2.0, alpha_value=2.0))
    layer.update(k[:, :, :2048 + 128].contiguous(), v[:, :, :2048 + 128].contiguous(), {"materialize_full_kv": False})
    for t in range(2048 + 128, S):
        layer.update(k[:, :, t:t + 1], v[:, :, t:t + 1], {"materialize_full_kv": False})
    assert layer._key_group_count == 32 and layer.keys.shape[2] == 150
    mask = torch.zeros(B, 1, 1, S)
    mask[0, ..., :200] = torch.finfo(torch.bfloat16).min           # left padding
    mask[7, ..., 1990:2100] = -4.0                                  # across the packed / residual boundary
    mask[15, ..., S - 9:] = torch.finfo(torch.bfloat16).min        # the ragged last residual tile
    got = decode_attention(layer, q, 128 ** -0.5, mask.cuda(), out_dtype=torch.float32)
    rec = decode_attention_partial_packed(layer, q, 128 ** -0.5, mask.cuda())        # [B, H, D + 2] = acc, m, l
    for i, r in enumerate(rows):
        ref = oracle.OracleCacheLayer(bits=bits, group=64, residual=128, alpha_key=2.0, alpha_value=2.0)
        ref.append(kc[i:i + 1, :, :2048 + 128].contiguous(), vc[i:i + 1, :, :2048 + 128].contiguous())
        for t in range(2048 + 128, S):
            ref.append(kc[i:i + 1, :, t:t + 1].contiguous(), vc[i:i + 1, :, t:t + 1].contiguous())
        want = oracle.decode_attention_oracle(qc[i:i + 1], ref, 128 ** -0.5, gqa, mask=mask[r:r + 1], compute_dtype=torch.float32)
        err = (got[r:r + 1].cpu() - want).abs().max().item()
        assert err <= TOL, (r, err)
        pr = rec[r].cpu()
        from_triple = (pr[:, :128] / pr[:, 129:130]).view(1, 1, H, 128)
        assert (from_triple - want).abs().max().item() <= TOL, r
