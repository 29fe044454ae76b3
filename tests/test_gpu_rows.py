"""GPU: row quantizer / dequantizer through the C-ABI against golden vectors and the oracle."""
import numpy as np
import pytest
import torch

from conftest import DTYPES, bits16, from_bits16

pytestmark = pytest.mark.gpu


def _meta_arr(t):
    t = t.cpu()
    return t.numpy() if t.dtype == torch.float32 else bits16(t)


def test_quantize_rows_golden_bit_exact(golden):
    import muzero_b200 as mz
    g = golden.rows_quant
    keys = [k[:-7] for k in g.files if k.endswith("_packed")]
    assert len(keys) > 100
    for key in keys:
        grp, dname, b, a, m = key.split("_")
        group, bits, alpha, mname = int(grp[1:]), int(b[1:]), float(a[1:]), m[1:]
        x = torch.from_numpy(g[f"x_g{group}"]).to(DTYPES[dname]).cuda()
        pq, mn, sc = mz.quantize_rows(x, bits, alpha, 1e-8, DTYPES[mname])
        ok = np.ones(x.shape[0], dtype=bool)
        if dname == "fp16":   # zero range in fp16 -> NaN in the reference; codes unspecified there
            ok = _meta_arr(sc).reshape(-1) != 0
        assert np.array_equal(pq.cpu().numpy()[ok], g[key + "_packed"][ok]), key
        assert np.array_equal(_meta_arr(mn), g[key + "_mn"]), key
        assert np.array_equal(_meta_arr(sc), g[key + "_scale"]), key


def test_dequantize_rows_golden_bit_exact(golden):
    import muzero_b200 as mz
    g, d = golden.rows_quant, golden.rows_dequant
    for key in [k[:-4] for k in d.files if k.endswith("_f32")]:
        grp, dname, b, a, m = key.split("_")
        group, bits, alpha = int(grp[1:]), int(b[1:]), float(a[1:])
        pq = torch.from_numpy(g[key + "_packed"]).cuda()
        mn = from_bits16(g[key + "_mn"], torch.float16).cuda()
        sc = from_bits16(g[key + "_scale"], torch.float16).cuda()
        o32 = mz.dequantize_rows(pq, mn, sc, bits, alpha, group, torch.float32)
        obf = mz.dequantize_rows(pq, mn, sc, bits, alpha, group, torch.bfloat16)
        assert np.array_equal(o32.cpu().numpy().view(np.uint32), d[key + "_f32"].view(np.uint32)), key
        assert np.array_equal(bits16(obf), d[key + "_bf16"]), key


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_quantize_rows_vs_oracle_large(oracle, dtype, bits):
    import muzero_b200 as mz
    gen = torch.Generator().manual_seed(100 + bits)
    for group, alpha in ((64, 2.0), (32, 4.0), (128, 16.0)):
        x = (torch.randn(4096, group, generator=gen) * torch.exp(torch.randn(4096, 1, generator=gen))).to(dtype)
        if dtype == torch.float16:
            x = x.clamp(-60000, 60000)
        ref = oracle.quantize_rows_oracle(x, bits, alpha, 1e-8, torch.float16)
        got = mz.quantize_rows(x.cuda(), bits, alpha, 1e-8, torch.float16)
        assert torch.equal(got[0].cpu(), ref[0])
        assert np.array_equal(bits16(got[1]), bits16(ref[1])) and np.array_equal(bits16(got[2]), bits16(ref[2]))
        back = mz.dequantize_rows(got[0], got[1], got[2], bits, alpha, group, torch.float32).cpu()
        want = oracle.dequantize_rows_oracle(ref[0], ref[1], ref[2], bits, alpha, group, torch.float32)
        assert torch.equal(back, want)


@pytest.mark.parametrize("group", [8, 24, 100, 256])
def test_odd_group_sizes(oracle, group):
    import muzero_b200 as mz
    gen = torch.Generator().manual_seed(group)
    x = torch.randn(257, group, generator=gen).to(torch.bfloat16)
    for bits in (1, 3, 4, 7):
        ref = oracle.quantize_rows_oracle(x, bits, 2.0, 1e-8, torch.float16)
        got = mz.quantize_rows(x.cuda(), bits, 2.0, 1e-8, torch.float16)
        assert torch.equal(got[0].cpu(), ref[0]), (group, bits)
        assert np.array_equal(bits16(got[2]), bits16(ref[2]))
        back = mz.dequantize_rows(got[0], got[1], got[2], bits, 2.0, group, torch.bfloat16).cpu()
        want = oracle.dequantize_rows_oracle(ref[0], ref[1], ref[2], bits, 2.0, group, torch.bfloat16)
        assert np.array_equal(bits16(back), bits16(want))


def test_reference_quantizer_suite_thresholds():
    """The reference's own unit tests for this module (tests/test_quantizer.py), on the CUDA path."""
    import muzero_b200 as mz
    torch.manual_seed(42)
    flat = torch.randn(256, 64, device="cuda", dtype=torch.float32)
    for bits, thr in ((2, 0.35), (4, 0.015), (8, 1e-4)):
        pq, mn, sc = mz.quantize_rows(flat, bits, 2.0, 1e-8, torch.float16)
        assert pq.shape == (256, 64 * bits // 8) and mn.shape == (256, 1) and sc.shape == (256, 1)
        recon = mz.dequantize_rows(pq, mn, sc, bits, 2.0, 64, torch.float32)
        assert ((flat - recon) ** 2).mean().item() < thr
    t = torch.randn(4, 8, 64, 128, device="cuda")
    assert mz.select_alpha(t, bits=4, q_group_size=64, kind="key") == 2.0
    for bits, kind in ((1, "key"), (2, "value"), (8, "key")):
        a = mz.select_alpha(torch.randn(2, 4, 32, 64, device="cuda"), bits=bits, q_group_size=32, kind=kind)
        assert isinstance(a, float) and a > 0
    k = torch.randn(1, 8, 256, 128, device="cuda", dtype=torch.float16)
    v = torch.randn(1, 8, 256, 128, device="cuda", dtype=torch.float16)
    rk, rv = mz.roundtrip(k, v, bits=4, q_group_size=64)
    assert rk.shape == k.shape and rv.dtype == v.dtype
    cos = torch.nn.functional.cosine_similarity
    assert cos(k.reshape(1, -1).float(), rk.reshape(1, -1).float()).item() > 0.99
    assert cos(v.reshape(1, -1).float(), rv.reshape(1, -1).float()).item() > 0.99
    ones = torch.ones(64, 64, device="cuda")
    pq, mn, sc = mz.quantize_rows(ones, 4, 2.0, 1e-8, torch.float16)
    rec = mz.dequantize_rows(pq, mn, sc, 4, 2.0, 64, torch.float32)
    assert not torch.isnan(rec).any() and not torch.isinf(rec).any()
