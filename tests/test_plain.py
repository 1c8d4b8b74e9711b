"""The plain implementation itself (no GPU): against the committed outputs of
the reference's model code, and properties of the parts the reference lacks."""

import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama
from golden.make_golden import golden_tokens, golden_weights

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_matches_reference_outputs(name):
    meta = json.loads((GOLDEN / f"golden_{name}.json").read_text())
    config = meta["config"]
    weights = golden_weights(config, meta["seed"])
    assert golden_tokens(config, meta["seed"], len(meta["tokens"])) == meta["tokens"]
    ref = torch.from_numpy(np.fromfile(GOLDEN / f"golden_{name}.f32", dtype="<f4").reshape(len(meta["tokens"]), -1).copy())
    got = plain_llama.forward_logits(weights, config, meta["tokens"])
    assert float((got - ref).abs().max()) < 2e-6 * max(1.0, float(ref.abs().max()))


def test_llama3_scaling_properties():
    s = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64)
    f = plain_llama.rope_inv_freq(32, 500000.0)
    g = plain_llama.llama3_scale_inv_freq(f, s)
    wavelen = 2 * math.pi / f
    short, long_ = wavelen < 64 / 4.0, wavelen > 64 / 1.0
    assert short.any() and long_.any() and (~short & ~long_).any()
    assert torch.equal(g[short], f[short])                              # high frequencies untouched
    assert torch.allclose(g[long_], f[long_] / 8.0)                     # low frequencies divided by the factor
    mid = ~short & ~long_
    assert ((g[mid] < f[mid]) & (g[mid] > f[mid] / 8.0)).all()          # a blend between
    assert (g[:-1] >= g[1:]).all()                                       # still monotone


# llama3 frequency scaling at the parameters of the tiny-B, Llama-3.2-1B and Llama-3.2-3B configurations: which
# frequencies are kept, which divided by the factor, and the blended ones to twelve digits.  The figures were worked
# out once at 50 decimal digits from the published rule, stated in periods per original context (c = orig * f / 2 pi:
# c > high keeps f, c < low gives f / factor, else t = (c - low) / (high - low) and (1 - t) f / factor + t f), which is
# a third way of writing it beside the product's and the plain implementation's.  The reference has no such scaling
# (engine/layers.py:57-79 builds unscaled tables), and installed packages' model code is no source for this repository.
LLAMA3_PINS = {
    "tiny-b": (dict(theta=500000.0, head_dim=32, factor=8.0, low=1.0, high=4.0, orig=64), 2, 13,
               {2: 7.940300917921e-2, 15: 5.677088100760e-7}),
    "llama-3.2-1b": (dict(theta=500000.0, head_dim=64, factor=32.0, low=1.0, high=4.0, orig=8192), 15, 14,
                     {15: 1.290547928209e-3, 16: 4.295567965594e-4, 17: 9.708287802628e-5, 31: 9.418306725435e-8}),
    "llama-3.2-3b": (dict(theta=500000.0, head_dim=128, factor=32.0, low=1.0, high=4.0, orig=8192), 29, 29,
                     {29: 2.118406996780e-3, 30: 1.290547928209e-3, 31: 7.625412033564e-4, 32: 4.295567965594e-4,
                      33: 2.227635014685e-4, 34: 9.708287802628e-5, 63: 7.672314972286e-8}),
}


@pytest.mark.parametrize("name", sorted(LLAMA3_PINS))
def test_llama3_scaling_is_pinned_to_worked_out_figures(name):
    from inf_engine_b200.config import get_preset
    from inf_engine_b200.parts import rotary_inv_freq

    a, n_kept, n_divided, pins = LLAMA3_PINS[name]
    cfg = get_preset(name)
    s = cfg.rope_scaling
    assert (cfg.rope_theta, cfg.head_dim, s.factor, s.low_freq_factor, s.high_freq_factor,
            s.original_max_position_embeddings) == (a["theta"], a["head_dim"], a["factor"], a["low"], a["high"], a["orig"])
    product = rotary_inv_freq(cfg.model_spec().layers[0].mixer.position).double()
    base = plain_llama.rope_inv_freq(a["head_dim"], a["theta"])
    plain = plain_llama.llama3_scale_inv_freq(base, dict(factor=a["factor"], low_freq_factor=a["low"],
                                                         high_freq_factor=a["high"],
                                                         original_max_position_embeddings=a["orig"])).double()
    # the third formulation, in float64
    third = []
    for i in range(a["head_dim"] // 2):
        f = a["theta"] ** (-2.0 * i / a["head_dim"])
        c = a["orig"] * f / (2.0 * math.pi)
        t = (c - a["low"]) / (a["high"] - a["low"])
        third.append(f if c > a["high"] else f / a["factor"] if c < a["low"] else (1.0 - t) * f / a["factor"] + t * f)
    third = torch.tensor(third, dtype=torch.float64)
    for got in (product, plain):
        assert float(((got - third).abs() / third).max()) < 3e-7          # float32 tables against float64
        assert int((got == base.double()).sum()) == n_kept
        assert int(((got * a["factor"] - base.double()).abs() / base.double() < 1e-6).sum()) == n_divided
        for i, want in pins.items():
            assert abs(float(got[i]) - want) / want < 3e-7, (name, i, float(got[i]), want)
    for i, want in pins.items():
        assert abs(float(third[i]) - want) / want < 1e-11


def test_product_rope_tables_equal_the_plain_ones():
    from helpers import TINY_A, TINY_B
    from inf_engine_b200.config import parse_config_dict
    from inf_engine_b200.parts import rotary_tables

    for d in (TINY_A, TINY_B):
        spec = parse_config_dict(d).model_spec().layers[0].mixer.position
        cos, sin = rotary_tables(spec)
        pc, ps = plain_llama.rope_tables(d, d["max_position_embeddings"])
        half = d["head_dim"] // 2
        assert torch.equal(cos, pc[:, :half]) and torch.equal(sin, ps[:, :half])


def test_window_masks_old_keys():
    torch.manual_seed(0)
    cfg = dict(hidden_size=32, num_attention_heads=2, num_key_value_heads=1, head_dim=16)
    w = [torch.randn(32, 32) * 0.2, torch.randn(16, 32) * 0.2, torch.randn(16, 32) * 0.2, torch.randn(32, 32) * 0.2]
    h = torch.randn(12, 32)
    cos, sin = plain_llama.rope_tables(dict(cfg, rope_theta=10000.0), 12)
    full = plain_llama.attention(h, *w, cfg, cos, sin)
    win = plain_llama.attention(h, *w, cfg, cos, sin, window=4)
    assert torch.allclose(full[:4], win[:4], atol=1e-6) and not torch.allclose(full[8:], win[8:], atol=1e-4)
    # moving a token that the window has passed changes nothing
    h2 = h.clone()
    h2[0] += 3.0
    win2 = plain_llama.attention(h2, *w, cfg, cos, sin, window=4)
    assert torch.allclose(win[4:], win2[4:], atol=1e-6)


def test_sampling_filters():
    logits = torch.tensor([2.0, 1.0, 0.5, 1.0, -1.0])
    assert plain_llama.top_k_filter(logits, 2).isinf().tolist() == [False, False, True, False, True]   # ties kept
    assert plain_llama.top_k_filter(logits, 0).isinf().sum() == 4                                       # k clamps to 1
    p = torch.softmax(logits, -1)
    kept = ~plain_llama.top_p_filter(logits, float(p[0]) + 1e-4).isinf()
    assert kept[0] and kept.sum() == 2                                                                   # crosses p at the second
    assert (~plain_llama.top_p_filter(logits, 1e-9).isinf()).sum() == 1                                  # top-1 always stays
    out = plain_llama.apply_repetition_penalty(logits, [0, 4, 4, 0], 2.0)
    assert out.tolist() == [1.0, 1.0, 0.5, 1.0, -2.0]
    d = plain_llama.filtered_distribution(logits, "temperature", temperature=0.5)
    assert torch.allclose(d, torch.softmax(logits / 0.5, -1))
    assert plain_llama.filtered_distribution(logits, "greedy").tolist() == [1, 0, 0, 0, 0]
