"""GPU: the plug-in path end to end — patch_transformers() + model.generate(cache_implementation=
"mu_zero_4bit") on a random-init Qwen3-architecture decoder.

Checks that are robust on random-init weights (whose top-2 logit margins are within rounding
noise, so free-running token identity is not):
  * the fused decode path really runs (decode statistics, one call per layer per step);
  * teacher-forced comparison with the same cache read through the dense route
    (MUZERO_DISABLE_FUSED_DECODE=1: dequantized prefix + stock attention): identical packed
    codes, logits within bf16 noise, argmax agreement on all steps whose margin exceeds the noise;
  * the first index at which free-running greedy tokens leave the reference's own CPU run
    (tests/golden/generate_case.json) is reported, and the prefix before it must be non-trivial.
"""
import importlib.util
import json
import os

import pytest
import torch

from conftest import GOLDEN

pytestmark = pytest.mark.gpu


def _recipe_module():
    spec = importlib.util.spec_from_file_location("make_generate_golden", os.path.join(GOLDEN, "make_generate_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def setup():
    import muzero
    muzero.patch_transformers()
    gold = json.load(open(os.path.join(GOLDEN, "generate_case.json")))
    mk = _recipe_module()
    model = mk.build_model(gold["recipe"]).cuda()
    ids = mk.prompt_ids(gold["recipe"]).cuda()
    return muzero, gold, model, ids


def _generate(model, ids, gold, **extra):
    r = gold["recipe"]
    return model.generate(input_ids=ids, attention_mask=torch.ones_like(ids), max_new_tokens=r["new_tokens"], do_sample=False,
                          cache_implementation=r["cache_implementation"], cache_config=dict(r["cache_config"], **extra),
                          pad_token_id=0)[:, ids.shape[1]:]


def test_generate_runs_fused_path_and_is_deterministic(setup):
    muzero, gold, model, ids = setup
    r = gold["recipe"]
    muzero.reset_mu_zero_decode_stats()
    a = _generate(model, ids, gold, backend="cuda")
    st = muzero.get_mu_zero_decode_stats()
    layers, steps = r["model"]["num_hidden_layers"], r["new_tokens"] - 1
    assert st["calls"] == st["returns"] == layers * steps
    assert st["fused_qk_success"] == st["fused_av_success"] == layers * steps
    b = _generate(model, ids, gold, backend="cuda")
    assert torch.equal(a, b), "the kernels are deterministic: two runs must give identical tokens"
    ref = torch.tensor(gold["tokens"])
    same = (a.cpu() == ref)
    first_div = [int((~row).nonzero()[0]) if (~row).any() else row.numel() for row in same]
    print("first divergence from the reference's CPU run per sequence:", first_div)
    assert min(first_div) >= 1


def test_teacher_forced_fused_vs_dense_route(setup, monkeypatch):
    """Feed the same tokens through both routes step by step and compare logits."""
    muzero, gold, model, ids = setup
    r = gold["recipe"]
    forced = torch.tensor(gold["tokens"]).cuda()

    def run(disable_fused: bool):
        monkeypatch.setenv("MUZERO_DISABLE_FUSED_DECODE", "1" if disable_fused else "0")
        cache = muzero.MuZeroCache(muzero.MuZeroConfig(bits=4, **r["cache_config"]))
        cache.defer_prefill_quantization = True
        logits = []
        with torch.no_grad():
            out = model(input_ids=ids, past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1].float())
            for t in range(forced.shape[1] - 1):
                out = model(input_ids=forced[:, t:t + 1], past_key_values=cache, use_cache=True)
                logits.append(out.logits[:, -1].float())
        return torch.stack(logits, dim=1), cache

    fused, c1 = run(False)
    dense, c2 = run(True)
    for l1, l2 in zip(c1.layers, c2.layers):
        assert torch.equal(l1._packed_key_q, l2._packed_key_q) and torch.equal(l1._packed_value_q, l2._packed_value_q)
    diff = (fused - dense).abs().max().item()
    scale = dense.abs().max().item()
    assert diff <= 0.05 * max(scale, 1.0), (diff, scale)         # bf16 attention noise of the dense route
    top2 = dense.topk(2, dim=-1).values
    margin = top2[..., 0] - top2[..., 1]
    agree = fused.argmax(-1) == dense.argmax(-1)
    decisive = margin > 4 * diff
    assert bool(agree[decisive].all()), "argmax differs on a step whose margin exceeds the numerical noise"
    print(f"teacher-forced: max |dlogit| {diff:.4f} (logit scale {scale:.2f}), argmax agreement {agree.float().mean().item():.3f}")
