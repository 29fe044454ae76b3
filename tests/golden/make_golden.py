"""Generate the golden fixtures in this folder from the reference itself.

Run where the reference checkout is available (it is imported read-only and
run on CPU through its own ``backend="torch"`` path):

    python tests/golden/make_golden.py --reference /path/to/reference

Outputs (all small, committed):
  rows_quant.npz      seeded row inputs + packed codes / mn / scale of
                      ``_quantize_rows_torch`` for dtype x bits x alpha x group
  rows_dequant.npz    ``_dequantize_rows_torch`` outputs (fp32 and bf16) for the same codes
  expand_tables.npz   expm1 compander tables (bits<=6 in full, sha256 for 7/8)
  layer_cases.npz     MuZeroCacheLayer states (prefill flush, per-token decode
                      flush) and decode-attention outputs (as-is and fp32 evaluation)
  layer_cases_logq.npz  the same for ``logq_compatible_layout=True`` (``--only logq`` writes just these)
  config0.npz         batch 1 x 8 kv heads x 4096 tokens x head_dim 128 (4-bit, group 64, residual 128) at full size: sha256 of every store
                      tensor + the attention outputs
  alpha_cases.json    ``select_alpha`` results on the synthetic distributions

The GPU box has no reference checkout; tests only read the fixtures.
"""

from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import os
import sys
from types import SimpleNamespace

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _load_oracle():
    spec = importlib.util.spec_from_file_location("mz_oracle", os.path.join(ROOT, "oracle", "mz_oracle.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def sha(t: torch.Tensor) -> str:
    t = t.detach().contiguous().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.view(torch.int16)
    return hashlib.sha256(t.numpy().tobytes()).hexdigest()


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16)


def row_inputs(n_rows: int, group: int, seed: int) -> torch.Tensor:
    """fp32 master rows: a mix of the shapes a KV cache produces."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(n_rows, group, generator=gen)
    k = n_rows // 8
    x[0 * k:1 * k] *= torch.exp(torch.randn(k, 1, generator=gen) * 1.5)       # outlier rows
    x[1 * k:2 * k] = x[1 * k:2 * k].abs() + 0.25                               # all positive
    x[2 * k:3 * k] = -x[2 * k:3 * k].abs() - 0.5                               # all negative
    x[3 * k:4 * k] *= 1e-3                                                     # tiny range
    x[4 * k:5 * k] += 3.0                                                      # shifted
    x[5 * k] = 1.0                                                             # constant row
    x[5 * k + 1] = -2.5
    x[5 * k + 2, 1:] = 0.0                                                     # one spike
    return x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MUZERO_REFERENCE"), required="MUZERO_REFERENCE" not in os.environ,
                    help="path of the reference checkout (or set MUZERO_REFERENCE)")
    ap.add_argument("--only", default="all", choices=["all", "logq"], help="logq: write just layer_cases_logq.*")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import muzero  # the reference
    from muzero.quantizer import _quantize_rows_torch, _dequantize_rows_torch, select_alpha
    from muzero.cache.layer import MuZeroCacheLayer
    from muzero.cache.attention import mu_zero_decode_attention_forward
    from muzero.config import MuZeroConfig
    assert os.path.realpath(muzero.__file__).startswith(os.path.realpath(args.reference))
    orc = _load_oracle()
    torch.set_num_threads(max(1, torch.get_num_threads()))

    # ------------------------------------------------------------------ rows
    dtypes = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
    metas = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
    quant = {}
    deq = {}
    for group in (32, 64, 128):
        master = row_inputs(64, group, seed=1000 + group)
        quant[f"x_g{group}"] = master.numpy()
        for dname, dt in dtypes.items():
            x = master.to(dt)
            for bits in range(1, 9):
                for alpha in (2.0, 4.0, 16.0):
                    if group != 64 and alpha != 2.0 and bits not in (1, 8):
                        continue
                    for mname, mt in metas.items():
                        if mname != "fp16" and not (group == 64 and alpha == 2.0 and dname == "bf16"):
                            continue
                        pq, mn, sc = _quantize_rows_torch(x, bits, alpha, 1e-8, mt)
                        key = f"g{group}_{dname}_b{bits}_a{int(alpha)}_m{mname}"
                        quant[key + "_packed"] = pq.numpy()
                        if mt == torch.float32:
                            quant[key + "_mn"] = mn.numpy()
                            quant[key + "_scale"] = sc.numpy()
                        else:
                            quant[key + "_mn"] = bits16(mn)
                            quant[key + "_scale"] = bits16(sc)
                        if dname == "bf16" and mname == "fp16" and group == 64:
                            # skip degenerate rows (zero range in fp16 meta -> NaN in the reference)
                            out32 = _dequantize_rows_torch(pq, mn, sc, bits, alpha, group, torch.float32, 1e-8)
                            outbf = _dequantize_rows_torch(pq, mn, sc, bits, alpha, group, torch.bfloat16, 1e-8)
                            deq[key + "_f32"] = out32.numpy()
                            deq[key + "_bf16"] = bits16(outbf)
    if args.only == "all":
        np.savez_compressed(os.path.join(HERE, "rows_quant.npz"), **quant)
        np.savez_compressed(os.path.join(HERE, "rows_dequant.npz"), **deq)

    # ---------------------------------------------------------------- tables
    tabs = {}
    for bits in range(1, 9):
        for alpha in (2.0, 4.0, 16.0):
            top = 2 ** bits - 1
            lb = torch.log1p(torch.tensor(alpha, dtype=torch.float32))
            den = torch.arange(0, top + 1, dtype=torch.float32).clamp_min(1.0).view(-1, 1)
            num = torch.arange(0, top + 1, dtype=torch.float32).view(1, -1)
            t = torch.expm1((num / den).clamp(0.0, 1.0) * lb) / alpha
            if bits <= 6:
                tabs[f"b{bits}_a{int(alpha)}"] = t.numpy()
            else:
                tabs[f"b{bits}_a{int(alpha)}_sha"] = np.frombuffer(bytes.fromhex(sha(t)), dtype=np.uint8)
    if args.only == "all":
        np.savez_compressed(os.path.join(HERE, "expand_tables.npz"), **tabs)

    # ----------------------------------------------------------- layer cases
    def ref_layer(bits, group, residual, **kw):
        return MuZeroCacheLayer(MuZeroConfig(bits=bits, q_group_size=group, residual_length=residual,
                                             backend="torch", **kw))

    def attn(layer, q, gqa, fp32):
        mod = SimpleNamespace(num_key_value_groups=gqa)
        if fp32:
            saved = (layer.dtype, layer.keys, layer.values)
            layer.dtype = torch.float32
            layer.keys, layer.values = layer.keys.float(), layer.values.float()
            out, _ = mu_zero_decode_attention_forward(mod, q.float(), None, q.shape[-1] ** -0.5,
                                                      layer.get_attention_state())
            layer.dtype, layer.keys, layer.values = saved
            return out
        out, _ = mu_zero_decode_attention_forward(mod, q, None, q.shape[-1] ** -0.5,
                                                  layer.get_attention_state())
        return out

    def store_dict(prefix, layer, out):
        out[prefix + "packed_k"] = layer._packed_key_q.numpy()
        out[prefix + "packed_v"] = layer._packed_value_q.numpy()
        for nm, t in (("k_mn", layer._key_mn), ("k_scale", layer._key_scale),
                      ("v_mn", layer._value_mn), ("v_scale", layer._value_scale)):
            out[prefix + nm] = t.numpy() if t.dtype == torch.float32 else bits16(t)
        out[prefix + "res_k"] = bits16(layer.keys)
        out[prefix + "res_v"] = bits16(layer.values)
        out[prefix + "alpha"] = np.array([layer._selected_alpha_key, layer._selected_alpha_value], dtype=np.float64)

    cases = {}
    meta = {}
    specs = [
        # name, bits, group, residual, B, KVH, H, S, D, decode steps, extra cfg
        ("c4g64", 4, 64, 128, 1, 2, 8, 512, 128, 0, {}),
        ("c2g64", 2, 64, 128, 2, 2, 8, 384, 128, 0, {}),
        ("c3g32", 3, 32, 64, 1, 2, 4, 300, 128, 0, {}),
        ("c8g128", 8, 128, 128, 1, 1, 4, 640, 128, 0, {}),
        ("c1g64", 1, 64, 64, 1, 2, 8, 256, 128, 0, {}),
        ("c7g64", 7, 64, 64, 1, 1, 2, 256, 128, 0, {}),
        ("c4g64_d64", 4, 64, 64, 1, 4, 4, 256, 64, 0, {}),
        ("c4g64_dec", 4, 64, 128, 1, 2, 8, 200, 128, 70, {}),
        ("c2g64_dec4g", 2, 64, 128, 1, 2, 8, 130, 128, 300, {"decode_flush_by_group": False}),
        ("c4g64_bf16meta", 4, 64, 128, 1, 2, 8, 256, 128, 0, {"amax_dtype": "bfloat16"}),
        ("c4g64_f32meta", 4, 64, 128, 1, 2, 8, 256, 128, 0, {"amax_dtype": "float32"}),
    ]
    logq_specs = [
        # the legacy layout: every value token beyond the residual length is flushed, keys flush by whole groups,
        # so the value prefix runs ahead of the key prefix by up to group-1 tokens
        ("c4g64_logq", 4, 64, 128, 1, 2, 8, 300, 128, 0, {"logq_compatible_layout": True}),
        ("c4g64_logq_dec", 4, 64, 128, 2, 2, 8, 200, 128, 90, {"logq_compatible_layout": True}),
        ("c2g32_logq_dec", 2, 32, 64, 1, 2, 4, 150, 128, 40, {"logq_compatible_layout": True}),
    ]
    if args.only == "logq":
        specs, stem = logq_specs, "layer_cases_logq"
    else:
        stem = "layer_cases"
    for (name, bits, group, residual, B, KVH, H, S, D, steps, extra) in specs:
        seed = abs(hash(name)) % 100000 if False else sum(ord(c) for c in name)
        k, v, q = orc.synth_kv(B, KVH, S + steps, D, H, seed=seed)
        layer = ref_layer(bits, group, residual, **extra)
        layer.update(k[:, :, :S].contiguous(), v[:, :, :S].contiguous(), {"materialize_full_kv": False})
        for i in range(steps):
            layer.update(k[:, :, S + i:S + i + 1].contiguous(), v[:, :, S + i:S + i + 1].contiguous(),
                         {"materialize_full_kv": False})
        store_dict(name + "/", layer, cases)
        cases[name + "/attn_asis"] = bits16(attn(layer, q, H // KVH, fp32=False))
        cases[name + "/attn_fp32"] = attn(layer, q, H // KVH, fp32=True).numpy()
        deq_sha = dict(k=sha(layer._dequantize_key_prefix().contiguous()),
                       v=sha(layer._dequantize_value_prefix().contiguous()))
        meta[name] = dict(bits=bits, group=group, residual=residual, B=B, KVH=KVH, H=H, S=S, D=D,
                          steps=steps, seed=seed, extra=extra,
                          input_sha=dict(k=sha(k), v=sha(v), q=sha(q)), deq_bf16_sha=deq_sha)
    np.savez_compressed(os.path.join(HERE, stem + ".npz"), **cases)
    with open(os.path.join(HERE, stem + ".json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    if args.only == "logq":
        print("wrote", stem)
        return

    # --------------------------------------------------------------- config 0
    cfg0 = {}
    k, v, q = orc.synth_kv(1, 8, 4096, 128, 32, seed=0)
    summary = {"input_sha": dict(k=sha(k), v=sha(v), q=sha(q))}
    for bits in (4, 2):
        layer = ref_layer(bits, 64, 128)
        layer.update(k, v, {"materialize_full_kv": False})
        summary[f"b{bits}"] = dict(
            packed_k=sha(layer._packed_key_q), packed_v=sha(layer._packed_value_q),
            k_mn=sha(layer._key_mn), k_scale=sha(layer._key_scale),
            v_mn=sha(layer._value_mn), v_scale=sha(layer._value_scale),
            deq_k_bf16=sha(layer._dequantize_key_prefix().contiguous()),
            deq_v_bf16=sha(layer._dequantize_value_prefix().contiguous()),
            alpha=[layer._selected_alpha_key, layer._selected_alpha_value],
            shapes=dict(packed_k=list(layer._packed_key_q.shape), packed_v=list(layer._packed_value_q.shape)),
        )
        cfg0[f"b{bits}_attn_asis"] = bits16(attn(layer, q, 4, fp32=False))
        cfg0[f"b{bits}_attn_fp32"] = attn(layer, q, 4, fp32=True).numpy()
    np.savez_compressed(os.path.join(HERE, "config0.npz"), **cfg0)
    with open(os.path.join(HERE, "config0.json"), "w") as f:
        json.dump(summary, f, indent=1, sort_keys=True)

    # ------------------------------------------------------------------ alpha
    alphas = {}
    k, v, _ = orc.synth_kv(2, 4, 1024, 128, 8, seed=7)
    for group in (32, 64, 128):
        kr = orc.key_rows(k, group)
        vr = orc.value_rows(v, group)
        for bits in (1, 2, 3, 4, 7, 8):
            alphas[f"key_rows_b{bits}_g{group}"] = select_alpha(kr, bits=bits, q_group_size=group, kind="key")
            alphas[f"value_rows_b{bits}_g{group}"] = select_alpha(vr, bits=bits, q_group_size=group, kind="value")
            alphas[f"key_4d_b{bits}_g{group}"] = select_alpha(k, bits=bits, q_group_size=group, kind="key")
            alphas[f"value_4d_b{bits}_g{group}"] = select_alpha(v, bits=bits, q_group_size=group, kind="value")
    heavy = torch.randn(4096, 64, generator=torch.Generator().manual_seed(3)) ** 3
    for bits in (1, 3, 8):
        alphas[f"heavy_key_b{bits}"] = select_alpha(heavy, bits=bits, q_group_size=64, kind="key")
        alphas[f"heavy_value_b{bits}"] = select_alpha(heavy, bits=bits, q_group_size=64, kind="value")
    with open(os.path.join(HERE, "alpha_cases.json"), "w") as f:
        json.dump(alphas, f, indent=1, sort_keys=True)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
