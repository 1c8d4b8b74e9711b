"""Checkpoint reading, the one error that lists what is wrong, precision policy,
and the random-weights mode (no GPU)."""

import json

import pytest
import torch

from helpers import TINY_A, TINY_B
from inf_engine_b200.config import parse_config_dict
from inf_engine_b200.parts import expected_tensors
from inf_engine_b200.weights import (
    CheckpointFormatError,
    WeightsError,
    kept_dtype,
    load_weights,
    open_checkpoint,
    write_random_model,
    write_safetensors,
)


def _folder(tmp_path, d, seed=3, store="bfloat16"):
    cfg = parse_config_dict(d)
    return cfg, write_random_model(cfg, seed, tmp_path / f"m{seed}{store}", store_dtype=store)


def test_container_round_trip_agrees_with_the_safetensors_package(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file

    t = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "c": torch.arange(6, dtype=torch.int64).view(2, 3),
         "d": torch.randn(2, 2).half()}
    write_safetensors(tmp_path / "model.safetensors", t, metadata={"k": "v"})
    with safe_open(str(tmp_path / "model.safetensors"), framework="pt") as f:
        for k in t:
            assert torch.equal(f.get_tensor(k), t[k])
    other = tmp_path / "other"
    other.mkdir()
    save_file(t, str(other / "model.safetensors"))
    mine = open_checkpoint(other)
    for k in t:
        assert mine[k].shape == tuple(t[k].shape) and torch.equal(mine[k].read(), t[k])


def test_sharded_checkpoint_and_missing_files(tmp_path):
    a, b = {"x": torch.ones(2, 2)}, {"y": torch.zeros(3)}
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", a)
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", b)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "model-00001-of-00002.safetensors", "y": "model-00002-of-00002.safetensors"}}))
    assert set(open_checkpoint(tmp_path)) == {"x", "y"}
    (tmp_path / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(FileNotFoundError, match="shard"):
        open_checkpoint(tmp_path)
    with pytest.raises(FileNotFoundError, match="not found"):
        open_checkpoint(tmp_path / "nowhere")
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(FileNotFoundError, match="no model.safetensors"):
        open_checkpoint(empty)


def test_malformed_container(tmp_path):
    (tmp_path / "model.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00not json at all!")
    with pytest.raises(CheckpointFormatError):
        open_checkpoint(tmp_path)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg, folder = _folder(tmp_path, TINY_B)
    stored = {k: v.read().clone() for k, v in open_checkpoint(folder).items()}
    stored.pop("model.layers.1.mlp.up_proj.weight")
    stored.pop("model.norm.weight")
    stored["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(4)
    stored["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(5, 120)
    bad = tmp_path / "bad"
    bad.mkdir()
    write_safetensors(bad / "model.safetensors", stored)
    spec = cfg.model_spec()
    with pytest.raises(WeightsError) as e:
        load_weights(bad, expected_tensors(spec), torch.bfloat16, "cpu", spec.optional_tensors)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.2.self_attn.k_proj.weight"]
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "expected (64, 120), found (5, 120)"):
        assert piece in text


def test_tied_checkpoint_may_carry_a_head(tmp_path):
    cfg, folder = _folder(tmp_path, TINY_A)
    stored = {k: v.read().clone() for k, v in open_checkpoint(folder).items()}
    stored["lm_head.weight"] = torch.zeros(256, 64)
    d = tmp_path / "tied"
    d.mkdir()
    write_safetensors(d / "model.safetensors", stored)
    spec = cfg.model_spec()
    out = load_weights(d, expected_tensors(spec), torch.float32, "cpu", spec.optional_tensors)
    assert "lm_head.weight" not in out       # the tie wins (engine/llama_weights.py:45-47)


def test_precision_policy():
    bf, f32 = torch.bfloat16, torch.float32
    assert kept_dtype(bf, bf) is bf and kept_dtype(torch.float16, bf) is bf
    assert kept_dtype(f32, bf) is f32            # a tensor stored in 32-bit stays so
    assert kept_dtype(bf, f32) is f32 and kept_dtype(f32, f32) is f32
    assert kept_dtype(torch.int64, bf) is torch.int32 and kept_dtype(torch.uint8, f32) is torch.int32


def test_loader_applies_the_policy(tmp_path):
    cfg, folder = _folder(tmp_path, TINY_A)
    stored = {k: v.read().clone() for k, v in open_checkpoint(folder).items()}
    stored["model.norm.weight"] = stored["model.norm.weight"].float()
    d = tmp_path / "mixed"
    d.mkdir()
    write_safetensors(d / "model.safetensors", stored)
    spec = cfg.model_spec()
    out = load_weights(d, expected_tensors(spec), torch.bfloat16, "cpu")
    assert out["model.norm.weight"].dtype is torch.float32
    assert out["model.embed_tokens.weight"].dtype is torch.bfloat16
    out = load_weights(d, expected_tensors(spec), torch.float32, "cpu")
    assert all(t.dtype is torch.float32 for t in out.values())


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    cfg, folder = _folder(tmp_path, TINY_B, seed=5)
    assert (folder / "config.json").is_file() and (folder / "model.safetensors").is_file()
    assert parse_config_dict(json.loads((folder / "config.json").read_text())) == cfg
    spec = cfg.model_spec()
    out = load_weights(folder, expected_tensors(spec), torch.float32, "cpu")
    assert set(out) == set(expected_tensors(spec))
    emb = out["model.embed_tokens.weight"]
    assert emb.shape == (389, 120) and 0.01 < float(emb.std()) < 0.03
    gain = out["model.layers.0.input_layernorm.weight"]
    assert 0.89 < float(gain.min()) and float(gain.max()) < 1.11 and float(gain.std()) > 0.01


def test_random_weights_depend_on_the_seed_only(tmp_path):
    _, a = _folder(tmp_path / "x", TINY_A, seed=7)
    _, b = _folder(tmp_path / "y", TINY_A, seed=7)
    _, c = _folder(tmp_path / "z", TINY_A, seed=8)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    _, f32 = _folder(tmp_path / "w", TINY_A, seed=7, store="float32")
    assert open_checkpoint(f32)["model.norm.weight"].dtype_tag == "F32"


def test_stored_rotary_frequencies_are_passed_over_and_reported(tmp_path):
    cfg, folder = _folder(tmp_path, TINY_A)
    stored = {k: v.read().clone() for k, v in open_checkpoint(folder).items()}
    stored["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    stored["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    d = tmp_path / "old_style"
    d.mkdir()
    write_safetensors(d / "model.safetensors", stored)
    spec = cfg.model_spec()
    with pytest.warns(UserWarning, match="2 stored buffers are not weights"):
        out = load_weights(d, expected_tensors(spec), torch.float32, "cpu", spec.optional_tensors)
    assert set(out) == set(expected_tensors(spec))
    # anything else that the model does not read is still an error
    stored["model.layers.0.self_attn.rotary_emb.other"] = torch.ones(8)
    write_safetensors(d / "model.safetensors", stored)
    with pytest.raises(WeightsError, match="rotary_emb.other"):
        load_weights(d, expected_tensors(spec), torch.float32, "cpu", spec.optional_tensors)


def test_only_declared_gains_are_drawn_as_gains():
    from inf_engine_b200.weights.loader import ExpectedTensor
    from inf_engine_b200.weights.random_init import random_tensors

    t = random_tensors({"gain": ExpectedTensor((4096,), init="gain"), "bias": ExpectedTensor((4096,)),
                        "matrix": ExpectedTensor((64, 64))}, seed=3, std=0.02, store_dtype="float32")
    assert abs(float(t["gain"].mean()) - 1.0) < 0.01 and float(t["gain"].min()) >= 0.9
    assert abs(float(t["bias"].mean())) < 0.005 and 0.015 < float(t["bias"].std()) < 0.025
    with pytest.raises(ValueError, match="unknown random initialisation"):
        random_tensors({"x": ExpectedTensor((4,), init="ones")}, seed=0)
