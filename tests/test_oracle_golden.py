"""CPU: the oracle restatement against the reference's own outputs (golden fixtures)."""
import hashlib

import numpy as np
import pytest
import torch

from conftest import DTYPES, bits16, from_bits16, sha


def _meta_arr(t):
    return t.numpy() if t.dtype == torch.float32 else bits16(t)


def test_pack_unpack_roundtrip(oracle):
    gen = torch.Generator().manual_seed(5)
    for bits in range(1, 9):
        for group in (8, 24, 32, 64, 100, 128):
            codes = torch.randint(0, 2 ** bits, (7, group), generator=gen).to(torch.uint8)
            packed = oracle.pack_codes(codes, bits)
            assert packed.shape == (7, (group * bits + 7) // 8)
            assert torch.equal(oracle.unpack_codes(packed, bits, group), codes)
    # known-answer: 4-bit codes 1,2,3,4 -> bytes 0x21 0x43 ; 2-bit 1,2,3,0 -> 0b00111001
    assert oracle.pack_codes(torch.tensor([[1, 2, 3, 4]], dtype=torch.uint8), 4).tolist() == [[0x21, 0x43]]
    assert oracle.pack_codes(torch.tensor([[1, 2, 3, 0]], dtype=torch.uint8), 2).tolist() == [[0b00111001]]
    # 3-bit codes 5,6 -> bits 101 011 (lsb first) -> 0b00110101
    assert oracle.pack_codes(torch.tensor([[5, 6]], dtype=torch.uint8), 3).tolist() == [[0b00110101]]


def test_quantize_rows_match_reference(oracle, golden):
    g = golden.rows_quant
    keys = [k[:-7] for k in g.files if k.endswith("_packed")]
    assert len(keys) > 100
    for key in keys:
        grp, dname, b, a, m = key.split("_")
        group, bits, alpha = int(grp[1:]), int(b[1:]), float(a[1:])
        x = torch.from_numpy(g[f"x_g{group}"]).to(DTYPES[dname])
        pq, mn, sc = oracle.quantize_rows_oracle(x, bits, alpha, 1e-8, DTYPES[m[1:]])
        assert np.array_equal(pq.numpy(), g[key + "_packed"]), key
        assert np.array_equal(_meta_arr(mn), g[key + "_mn"]), key
        assert np.array_equal(_meta_arr(sc), g[key + "_scale"]), key


def test_dequantize_rows_match_reference(oracle, golden):
    g, d = golden.rows_quant, golden.rows_dequant
    keys = [k[:-4] for k in d.files if k.endswith("_f32")]
    assert len(keys) == 24
    for key in keys:
        grp, dname, b, a, m = key.split("_")
        group, bits, alpha = int(grp[1:]), int(b[1:]), float(a[1:])
        pq = torch.from_numpy(g[key + "_packed"])
        mn = from_bits16(g[key + "_mn"], torch.float16)
        sc = from_bits16(g[key + "_scale"], torch.float16)
        o32 = oracle.dequantize_rows_oracle(pq, mn, sc, bits, alpha, group, torch.float32)
        obf = oracle.dequantize_rows_oracle(pq, mn, sc, bits, alpha, group, torch.bfloat16)
        assert np.array_equal(o32.numpy().view(np.uint32), d[key + "_f32"].view(np.uint32)), key
        assert np.array_equal(bits16(obf), d[key + "_bf16"]), key


def test_expand_tables_match_reference(oracle, golden):
    for bits in range(1, 9):
        for alpha in (2.0, 4.0, 16.0):
            t = oracle.expand_table_oracle(bits, alpha)
            key = f"b{bits}_a{int(alpha)}"
            if bits <= 6:
                assert np.array_equal(t.numpy().view(np.uint32), golden.tables[key].view(np.uint32))
            else:
                assert sha(t) == bytes(golden.tables[key + "_sha"]).hex()


def test_select_alpha_matches_reference(oracle, golden):
    k, v, _ = oracle.synth_kv(2, 4, 1024, 128, 8, seed=7)
    for group in (32, 64, 128):
        kr, vr = oracle.key_rows(k, group), oracle.value_rows(v, group)
        for bits in (1, 2, 3, 4, 7, 8):
            a = golden.alpha
            assert oracle.select_alpha_oracle(kr, bits=bits, group=group, kind="key") == a[f"key_rows_b{bits}_g{group}"]
            assert oracle.select_alpha_oracle(vr, bits=bits, group=group, kind="value") == a[f"value_rows_b{bits}_g{group}"]
            assert oracle.select_alpha_oracle(k, bits=bits, group=group, kind="key") == a[f"key_4d_b{bits}_g{group}"]
            assert oracle.select_alpha_oracle(v, bits=bits, group=group, kind="value") == a[f"value_4d_b{bits}_g{group}"]
    heavy = torch.randn(4096, 64, generator=torch.Generator().manual_seed(3)) ** 3
    for bits in (1, 3, 8):
        assert oracle.select_alpha_oracle(heavy, bits=bits, group=64, kind="key") == golden.alpha[f"heavy_key_b{bits}"]
        assert oracle.select_alpha_oracle(heavy, bits=bits, group=64, kind="value") == golden.alpha[f"heavy_value_b{bits}"]
    assert set(golden.alpha.values()) > {2.0}, "fixture should exercise more than the default alpha"


def build_case(oracle, meta):
    """Replay one golden layer case through the oracle layer; returns (layer, q)."""
    md = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
    extra = meta["extra"]
    k, v, q = oracle.synth_kv(meta["B"], meta["KVH"], meta["S"] + meta["steps"], meta["D"], meta["H"], seed=meta["seed"])
    assert sha(k) == meta["input_sha"]["k"] and sha(v) == meta["input_sha"]["v"] and sha(q) == meta["input_sha"]["q"]
    layer = oracle.OracleCacheLayer(bits=meta["bits"], group=meta["group"], residual=meta["residual"],
                                    meta_dtype=md[extra.get("amax_dtype", "float16")],
                                    flush_by_group=extra.get("decode_flush_by_group", True),
                                    logq_layout=extra.get("logq_compatible_layout", False))
    S = meta["S"]
    layer.append(k[:, :, :S].contiguous(), v[:, :, :S].contiguous())
    for i in range(meta["steps"]):
        layer.append(k[:, :, S + i:S + i + 1].contiguous(), v[:, :, S + i:S + i + 1].contiguous())
    return layer, q


@pytest.mark.parametrize("name", ["c4g64", "c2g64", "c3g32", "c8g128", "c1g64", "c7g64", "c4g64_d64",
                                  "c4g64_dec", "c2g64_dec4g", "c4g64_bf16meta", "c4g64_f32meta"])
def test_layer_cases_match_reference(oracle, golden, name):
    _check_layer_case(oracle, golden.layer_meta[name], golden.layer, name)


@pytest.mark.parametrize("name", ["c4g64_logq", "c4g64_logq_dec", "c2g32_logq_dec"])
def test_logq_layout_cases_match_reference(oracle, golden, name):
    """`logq_compatible_layout=True`: the value prefix runs ahead of the key prefix."""
    g = golden.layer_logq
    assert g[name + "/packed_v"].shape[2] > g[name + "/packed_k"].shape[2] * golden.layer_logq_meta[name]["group"]
    _check_layer_case(oracle, golden.layer_logq_meta[name], g, name)


def _check_layer_case(oracle, meta, g, name):
    layer, q = build_case(oracle, meta)
    assert np.array_equal(layer.packed_k.numpy(), g[name + "/packed_k"])
    assert np.array_equal(layer.packed_v.numpy(), g[name + "/packed_v"])
    for nm in ("k_mn", "k_scale", "v_mn", "v_scale"):
        assert np.array_equal(_meta_arr(getattr(layer, nm)), g[f"{name}/{nm}"]), nm
    assert np.array_equal(bits16(layer.keys), g[name + "/res_k"])
    assert np.array_equal(bits16(layer.values), g[name + "/res_v"])
    assert [layer.alpha_key, layer.alpha_value] == list(g[name + "/alpha"])
    assert sha(layer.key_prefix(torch.bfloat16).contiguous()) == meta["deq_bf16_sha"]["k"]
    assert sha(layer.value_prefix(torch.bfloat16).contiguous()) == meta["deq_bf16_sha"]["v"]
    gqa = meta["H"] // meta["KVH"]
    scaling = meta["D"] ** -0.5
    out32 = oracle.decode_attention_oracle(q, layer, scaling, gqa, compute_dtype=torch.float32)
    ref32 = torch.from_numpy(g[name + "/attn_fp32"])
    assert out32.shape == ref32.shape
    assert (out32 - ref32).abs().max().item() < 2e-5      # same math, fp32 summation order only
    out_asis = oracle.decode_attention_oracle(q, layer, scaling, gqa)
    ref_asis = from_bits16(g[name + "/attn_asis"], torch.bfloat16).float()
    # bf16 GEMM summation order differs between chunkings; stays within bf16 noise
    assert (out_asis.float() - ref_asis).abs().max().item() < 6e-2


def test_config0_full_size(oracle, golden):
    meta = golden.config0_meta
    k, v, q = oracle.synth_kv(1, 8, 4096, 128, 32, seed=0)
    assert sha(k) == meta["input_sha"]["k"] and sha(v) == meta["input_sha"]["v"]
    for bits in (4, 2):
        layer = oracle.OracleCacheLayer(bits=bits, group=64, residual=128)
        layer.append(k, v)
        m = meta[f"b{bits}"]
        assert list(layer.packed_k.shape) == m["shapes"]["packed_k"] == [1, 8, 62, 128, 64 * bits // 8]
        assert sha(layer.packed_k) == m["packed_k"] and sha(layer.packed_v) == m["packed_v"]
        assert sha(layer.k_mn) == m["k_mn"] and sha(layer.k_scale) == m["k_scale"]
        assert sha(layer.v_mn) == m["v_mn"] and sha(layer.v_scale) == m["v_scale"]
        assert sha(layer.key_prefix(torch.bfloat16).contiguous()) == m["deq_k_bf16"]
        assert sha(layer.value_prefix(torch.bfloat16).contiguous()) == m["deq_v_bf16"]
        out = oracle.decode_attention_oracle(q, layer, 128 ** -0.5, 4, compute_dtype=torch.float32)
        ref = torch.from_numpy(golden.config0[f"b{bits}_attn_fp32"])
        assert (out - ref).abs().max().item() < 2e-5


def test_lse_merge_equals_monolithic(oracle):
    k, v, q = oracle.synth_kv(2, 2, 300, 64, 8, seed=11)
    m, l, acc = oracle.attention_partial_oracle(q, k, v, 0.125, 4)
    whole = acc / l.unsqueeze(-1)
    cuts = [0, 64, 65, 200, 300]
    parts = [oracle.attention_partial_oracle(q, k[:, :, a:b], v[:, :, a:b], 0.125, 4) for a, b in zip(cuts, cuts[1:])]
    merged = oracle.lse_merge_oracle([p[0] for p in parts], [p[1] for p in parts], [p[2] for p in parts])
    assert (merged - whole).abs().max().item() < 1e-5
