"""Golden greedy tokens of the reference itself: a random-init Qwen3-architecture decoder run on
CPU through the reference's `patch_transformers()` + `generate(cache_implementation="mu_zero_4bit",
backend="torch")`.  Writes generate_case.json (token ids + the model/prompt recipe) and generate_logits.npz
(the reference's fp32 logits of every generated position, [batch, new_tokens, vocab]).

    python tests/golden/make_generate_golden.py [--reference /path/to/reference]
"""
import argparse
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))

MODEL = dict(num_hidden_layers=2, hidden_size=256, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
             intermediate_size=512, vocab_size=1024, max_position_embeddings=2048, rms_norm_eps=1e-6,
             rope_theta=1e6, tie_word_embeddings=False)
RECIPE = dict(model=MODEL, weight_seed=0, weight_std=0.02, prompt_seed=1, batch=2, prompt_len=300, new_tokens=96,
              cache_implementation="mu_zero_4bit", cache_config={"q_group_size": 64, "residual_length": 128})


def build_model(recipe, dtype=torch.bfloat16):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    cfg = Qwen3Config(**recipe["model"])
    torch.manual_seed(recipe["weight_seed"])
    model = Qwen3ForCausalLM(cfg)
    gen = torch.Generator().manual_seed(recipe["weight_seed"])
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() > 1:
                p.copy_(torch.randn(p.shape, generator=gen) * recipe["weight_std"])
    return model.to(dtype).eval()


def prompt_ids(recipe):
    gen = torch.Generator().manual_seed(recipe["prompt_seed"])
    return torch.randint(0, recipe["model"]["vocab_size"], (recipe["batch"], recipe["prompt_len"]), generator=gen)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MUZERO_REFERENCE"), required="MUZERO_REFERENCE" not in os.environ,
                    help="path of the reference checkout (or set MUZERO_REFERENCE)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import muzero
    assert os.path.realpath(muzero.__file__).startswith(os.path.realpath(args.reference))
    muzero.patch_transformers()
    model = build_model(RECIPE)
    ids = prompt_ids(RECIPE)
    cfg = dict(RECIPE["cache_config"], backend="torch")
    out = model.generate(input_ids=ids, attention_mask=torch.ones_like(ids), max_new_tokens=RECIPE["new_tokens"],
                         do_sample=False, cache_implementation=RECIPE["cache_implementation"], cache_config=cfg,
                         pad_token_id=0, output_logits=True, return_dict_in_generate=True)
    stats = muzero.get_mu_zero_decode_stats()
    logits = torch.stack([x.float() for x in out.logits], dim=1)          # [batch, new_tokens, vocab]
    out = out.sequences
    import numpy as np
    np.savez_compressed(os.path.join(HERE, "generate_logits.npz"), logits=logits.numpy())
    result = dict(recipe=RECIPE, tokens=out[:, ids.shape[1]:].tolist(), reference_decode_stats=stats,
                  torch=torch.__version__)
    with open(os.path.join(HERE, "generate_case.json"), "w") as f:
        json.dump(result, f, indent=1)
    print("tokens[0][:16] =", result["tokens"][0][:16], "stats", stats)


if __name__ == "__main__":
    main()
