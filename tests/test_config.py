"""Configuration and registry (no GPU)."""

import json

import pytest

from helpers import TINY_A, TINY_B
from inf_engine_b200.config import (
    ARCHITECTURES,
    AttentionSpec,
    ConfigError,
    GatedMLPSpec,
    LlamaConfig,
    detect_config,
    get_llama_config,
    get_preset,
    parse_config_dict,
    preset_names,
    register_architecture,
)


def test_reads_every_size_from_config_json():
    cfg = parse_config_dict(TINY_B)
    assert isinstance(cfg, LlamaConfig)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 120, 6, 2)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (32, 328, 389)
    assert cfg.rope_theta == 500000.0 and cfg.rms_norm_eps == 1e-6 and not cfg.tie_word_embeddings
    assert cfg.rope_scaling.factor == 8.0 and cfg.rope_scaling.original_max_position_embeddings == 64
    # the reference's short names are aliases
    assert (cfg.n_layer, cfg.d_model, cfg.n_head, cfg.n_kv_heads, cfg.n_kv_groups, cfg.n_ctx, cfg.norm_eps) == \
        (3, 120, 6, 2, 3, 1024, 1e-6)


def test_head_dim_defaults_to_hidden_over_heads():
    d = dict(TINY_A)
    d.pop("head_dim")
    assert parse_config_dict(d).head_dim == 16
    d["hidden_size"] = 66
    with pytest.raises(ConfigError, match="not divisible"):
        parse_config_dict(d)


def test_optional_keys_take_their_defaults():
    d = {k: v for k, v in TINY_A.items() if k not in ("rope_theta", "rms_norm_eps", "tie_word_embeddings", "rope_scaling")}
    cfg = parse_config_dict(d)
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-5 and cfg.tie_word_embeddings is False
    assert cfg.rope_scaling is None


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "intermediate_size", "max_position_embeddings"])
def test_missing_required_key(key):
    d = dict(TINY_A)
    d.pop(key)
    with pytest.raises(ConfigError, match=key):
        parse_config_dict(d)


def test_validation_errors():
    with pytest.raises(ConfigError, match="num_key_value_heads"):
        parse_config_dict(dict(TINY_A, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="hidden_act"):
        parse_config_dict(dict(TINY_A, hidden_act="gelu"))
    with pytest.raises(ConfigError, match="rope_scaling"):
        parse_config_dict(dict(TINY_A, rope_scaling={"rope_type": "yarn", "factor": 2.0}))
    with pytest.raises(ConfigError, match="lacks key"):
        parse_config_dict(dict(TINY_A, rope_scaling={"rope_type": "llama3", "factor": 2.0}))
    with pytest.raises(ConfigError, match="bias"):
        parse_config_dict(dict(TINY_A, attention_bias=True))
    with pytest.raises(ConfigError, match="even"):
        parse_config_dict(dict(TINY_A, head_dim=15))


def test_unknown_architecture_lists_known_ones():
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        parse_config_dict(dict(TINY_A, architectures=["NoSuchModel"]))
    with pytest.raises(ConfigError, match="architectures"):
        parse_config_dict({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_registry_takes_another_architecture():
    class Toy:
        def __init__(self, d):
            self.d = d

    register_architecture("ToyForTests", Toy)
    try:
        assert isinstance(parse_config_dict({"architectures": ["ToyForTests"]}), Toy)
    finally:
        ARCHITECTURES.pop("ToyForTests")


def test_detect_config_reads_the_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert detect_config(tmp_path) == parse_config_dict(TINY_B)
    with pytest.raises(FileNotFoundError):
        detect_config(tmp_path / "nowhere")


def test_round_trip_through_config_json():
    for d in (TINY_A, TINY_B):
        cfg = parse_config_dict(d)
        assert parse_config_dict(json.loads(json.dumps(cfg.to_hf_dict()))) == cfg


def test_presets_have_the_reference_sizes():
    # engine/config.py:77-133
    assert {"llama-3.2-1b", "llama-3.2-3b", "smollm2-1.7b", "tiny-a", "tiny-b"} <= set(preset_names())
    c = get_llama_config("llama-3.2-1b")
    assert (c.n_layer, c.d_model, c.n_head, c.n_kv_heads, c.intermediate_size, c.vocab_size) == (16, 2048, 32, 8, 8192, 128256)
    assert c.tie_word_embeddings and c.rope_scaling.factor == 32.0
    c = get_preset("llama-3.2-3b")
    assert (c.n_layer, c.d_model, c.n_head, c.head_dim) == (28, 3072, 24, 128)
    c = get_preset("smollm2-1.7b")
    assert (c.n_layer, c.n_kv_heads, c.vocab_size, c.rope_theta, c.rope_scaling) == (24, 32, 49152, 130000.0, None)
    with pytest.raises(KeyError):
        get_preset("no-such-preset")


def test_model_spec_is_per_layer_data():
    cfg = parse_config_dict(TINY_B)
    spec = cfg.model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.head == "lm_head.weight" and parse_config_dict(TINY_A).model_spec().head is None
    for i, blk in enumerate(spec.layers):
        assert isinstance(blk.mixer, AttentionSpec) and isinstance(blk.feedforward, GatedMLPSpec)
        assert blk.mixer.q_proj == f"model.layers.{i}.self_attn.q_proj.weight"
        assert blk.mixer.head_dim == 32 and blk.mixer.n_kv_heads == 2 and blk.mixer.window is None
        assert blk.mixer_norm.eps == 1e-6 and blk.feedforward.intermediate == 328
        assert blk.mixer.position.theta == 500000.0 and blk.mixer.position.scaling.factor == 8.0


def test_a_config_without_rope_theta_means_ten_thousand():
    # checkpoints of this architecture written before the key existed rotate with theta = 10000; the 500000 of the
    # reference's presets (engine/config.py:42) is named by every preset file and is no default of the reader
    d = {k: v for k, v in TINY_B.items() if k != "rope_theta"}
    assert parse_config_dict(d).rope_theta == 10000.0
    assert parse_config_dict(d).model_spec().layers[0].mixer.position.theta == 10000.0
    for name in preset_names():
        assert get_preset(name).rope_theta in (10000.0, 130000.0, 500000.0)


def test_model_spec_names_its_top_level():
    from inf_engine_b200.parts import MODELS, DecoderModel

    spec = parse_config_dict(TINY_A).model_spec()
    assert spec.kind == "decoder" and MODELS["decoder"] is DecoderModel
