"""Compare the plain implementation with the reference project's own model code
on the CPU and write the small outputs that ``tests/test_plain.py`` checks.

Usage:  python tests/golden/make_golden.py --reference <checkout of waleedalfar/inf-engine>

The reference's ``engine.llama_model.LlamaModel`` (engine/llama_model.py:25-150)
is imported from the given checkout and run in float32 on the CPU on two tiny
random models.  For the model with llama3 frequency scaling the reference, which
has no such scaling, gets its ``rope_cos``/``rope_sin`` attributes
(engine/llama_model.py:42-43) overwritten with the plain implementation's tables;
the scaling formula itself is therefore not anchored by the reference.

Outputs (float32, little-endian, committed):
  golden_<name>.json      config.json dictionary, seed, token ids, max |plain - reference|
  golden_<name>.f32       the reference's logits [T, vocab]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import plain_llama  # noqa: E402

CONFIGS = {
    "tiny_a": dict(
        architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, intermediate_size=176, vocab_size=256, rope_theta=10000.0,
        rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=128,
        hidden_act="silu",
    ),
    "tiny_b": dict(
        architectures=["LlamaForCausalLM"], num_hidden_layers=3, hidden_size=128, num_attention_heads=4,
        num_key_value_heads=1, head_dim=32, intermediate_size=320, vocab_size=384, rope_theta=500000.0,
        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=64),
        rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=256, hidden_act="silu",
    ),
}
SEEDS = {"tiny_a": 0, "tiny_b": 1}
LENGTHS = {"tiny_a": 33, "tiny_b": 70}


def golden_weights(config: dict, seed: int) -> dict:
    """N(0, 0.02) matrices and 1+U(-0.1, 0.1) norm gains from one seeded generator,
    in a fixed order of tensor names."""
    g = torch.Generator().manual_seed(seed)
    d = config["hidden_size"]
    hd = config["head_dim"]
    H, Hk, I, V = (config["num_attention_heads"], config["num_key_value_heads"],
                   config["intermediate_size"], config["vocab_size"])

    def mat(r, c):
        return torch.randn(r, c, generator=g) * 0.02

    def gain(n):
        return 1.0 + (torch.rand(n, generator=g) * 0.2 - 0.1)

    w = {"model.embed_tokens.weight": mat(V, d)}
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = gain(d)
        w[p + "self_attn.q_proj.weight"] = mat(H * hd, d)
        w[p + "self_attn.k_proj.weight"] = mat(Hk * hd, d)
        w[p + "self_attn.v_proj.weight"] = mat(Hk * hd, d)
        w[p + "self_attn.o_proj.weight"] = mat(d, H * hd)
        w[p + "post_attention_layernorm.weight"] = gain(d)
        w[p + "mlp.gate_proj.weight"] = mat(I, d)
        w[p + "mlp.up_proj.weight"] = mat(I, d)
        w[p + "mlp.down_proj.weight"] = mat(d, I)
    w["model.norm.weight"] = gain(d)
    if not config["tie_word_embeddings"]:
        w["lm_head.weight"] = mat(V, d)
    return w


def golden_tokens(config: dict, seed: int, n: int) -> list[int]:
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, config["vocab_size"], (n,), generator=g).tolist()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from engine.config import LlamaConfig
    from engine.llama_model import LlamaModel
    from engine.llama_weights import LlamaWeights

    for name, config in CONFIGS.items():
        seed = SEEDS[name]
        weights = golden_weights(config, seed)
        tokens = golden_tokens(config, seed, LENGTHS[name])
        ref_cfg = LlamaConfig(
            name=name, vocab_size=config["vocab_size"], n_ctx=config["max_position_embeddings"],
            d_model=config["hidden_size"], n_layer=config["num_hidden_layers"],
            n_head=config["num_attention_heads"], n_kv_heads=config["num_key_value_heads"],
            intermediate_size=config["intermediate_size"], rope_theta=config["rope_theta"],
            norm_eps=config["rms_norm_eps"], tie_word_embeddings=config["tie_word_embeddings"],
            head_dim_override=config["head_dim"],
        )
        model = LlamaModel(LlamaWeights(dict(weights), ref_cfg), ref_cfg)
        if config["rope_scaling"]:
            cos, sin = plain_llama.rope_tables(config, config["max_position_embeddings"])
            model.rope_cos, model.rope_sin = cos, sin
        ref_logits = model.forward(torch.tensor([tokens]))[0].float()
        plain_logits = plain_llama.forward_logits(weights, config, tokens)
        diff = float((ref_logits - plain_logits).abs().max())
        scale = float(ref_logits.abs().max())
        print(f"{name}: T={len(tokens)} max|plain-reference|={diff:.3e} max|logit|={scale:.3e}")
        assert diff < 1e-5 * max(scale, 1.0), "plain implementation disagrees with the reference"
        (HERE / f"golden_{name}.json").write_text(json.dumps(
            {"config": config, "seed": seed, "tokens": tokens, "max_abs_diff_plain_vs_reference": diff,
             "max_abs_logit": scale}, indent=1))
        (HERE / f"golden_{name}.f32").write_bytes(ref_logits.contiguous().numpy().astype("<f4").tobytes())


if __name__ == "__main__":
    main()
