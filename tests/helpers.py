"""Shared test helpers: tiny configurations that differ in every size and
option, model folders in temporary places, and comparisons with the plain
implementation."""

from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_llama

# Two tiny Llama configurations that differ in every size and option: layers,
# width, head counts and groups, head size, a feed-forward width and a
# vocabulary that are no power of two, theta, scaling, eps, tied or not.
TINY_A = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
    num_key_value_heads=2, head_dim=16, intermediate_size=176, vocab_size=256, rope_theta=10000.0,
    rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=512,
    hidden_act="silu",
)
TINY_B = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=3, hidden_size=120, num_attention_heads=6,
    num_key_value_heads=2, head_dim=32, intermediate_size=328, vocab_size=389, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=64),
    rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1024, hidden_act="silu",
)
# a third one for sizes the other two miss: one kv head (every query head in one group), head size 48
TINY_C = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=1, hidden_size=96, num_attention_heads=3,
    num_key_value_heads=1, head_dim=48, intermediate_size=200, vocab_size=301, rope_theta=20000.0,
    rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=512,
    hidden_act="silu",
)
# head sizes 64 and 128 are the ones the tensor-core attention kernels are built for
TINY_D = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=192, num_attention_heads=6,
    num_key_value_heads=2, head_dim=64, intermediate_size=272, vocab_size=333, rope_theta=100000.0,
    rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=128),
    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024, hidden_act="silu",
)
TINY_E = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=136, num_attention_heads=2,
    num_key_value_heads=1, head_dim=128, intermediate_size=144, vocab_size=270, rope_theta=50000.0,
    rope_scaling=None, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1024,
    hidden_act="silu",
)
# widths that are multiples of 256, so that the engine's decode steps take the bulk-copy streaming product, the norm
# handed over between two products and (for portions of 128 rows and more) the tcgen05 product: the paths of the
# full-size models, here small enough for the plain implementation
TINY_F = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
    num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=1000, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=128),
    rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=2048, hidden_act="silu",
)
# as many kv heads as query heads (no grouping), heads of 64
TINY_G = dict(
    architectures=["LlamaForCausalLM"], num_hidden_layers=2, hidden_size=128, num_attention_heads=2,
    num_key_value_heads=2, head_dim=64, intermediate_size=192, vocab_size=300, rope_theta=130000.0,
    rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024,
    hidden_act="silu",
)
TINY = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_d": TINY_D, "tiny_e": TINY_E,
        "tiny_f": TINY_F, "tiny_g": TINY_G}
SEEDS = {"tiny_a": 0, "tiny_b": 1, "tiny_c": 2, "tiny_d": 3, "tiny_e": 4, "tiny_f": 5, "tiny_g": 6}
# the two tiny configurations exactly as the package's presets state them (weights N(0, 0.02), seeds 0 and 1)
PRESET_SEEDS = {"tiny-a": 0, "tiny-b": 1}


def make_model_dir(tmp: Path, name: str, store_dtype: str = "bfloat16", std: float = 0.05) -> Path:
    """Write a random model folder with the package's random-weights mode."""
    from inf_engine_b200.config import parse_config_dict
    from inf_engine_b200.weights import write_random_model

    if name in PRESET_SEEDS:
        from inf_engine_b200.config import get_preset
        cfg, seed, std = get_preset(name), PRESET_SEEDS[name], 0.02
    else:
        cfg, seed = parse_config_dict(TINY[name]), SEEDS[name]
    out = Path(tmp) / f"{name}_{store_dtype}"
    if not (out / "model.safetensors").is_file():
        write_random_model(cfg, seed, out, store_dtype=store_dtype, std=std)
    return out


def plain_inputs(model_dir: Path):
    """(config dict, float32 weights) of a model folder for the plain implementation,
    read with the ``safetensors`` package rather than with the product's reader."""
    from safetensors import safe_open

    config = json.loads((Path(model_dir) / "config.json").read_text())
    weights = {}
    with safe_open(str(Path(model_dir) / "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            weights[k] = f.get_tensor(k).float()
    return config, weights


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# Bounds against the plain implementation.
#   float32: only the order of sums differs: an absolute bound relative to the largest logit.
#   bfloat16: activations and cache are rounded to 8 bits of mantissa at every stage.  Per row, the norm of the
#   difference over the norm of the plain row measures that noise without being diluted by the vocabulary's largest
#   logit.  Measured on a B200 over every comparison of this suite: worst row 0.009 (widths up to 192), 0.013 (width
#   256), 0.011 (two layers of width 2,048 and 3,072); mean over a request's rows 0.007, 0.008, 0.009.  The faults the
#   bounds must catch show, on the tiny models: rope_theta doubled 0.078-0.25 at the worst row (0.028-0.12 on
#   average), two early tokens swapped 0.019-0.05 at the worst row, eps x 100 0.021-0.34.
F32_ABS = 2e-5
BF16_ROW_MAX = 2.0e-2
BF16_ROW_MEAN = 1.2e-2
BF16_NEAR_TIE = 2.5e-2      # a row may choose another token only if the plain logits of the two are this close (x scale)
STATS: list[dict] = []      # what every comparison measured, for whoever wants to look (conftest can write it out)


def tolerance(dtype: str, ref: torch.Tensor) -> float:
    """Largest absolute logit difference allowed in float32 (summation order only)."""
    assert dtype == "float32"
    return F32_ABS * max(float(ref.abs().max()), 1.0)


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "", noise: float = 1.0) -> None:
    """``noise`` scales the bfloat16 bounds for a model that is built to amplify rounding (scores made ``noise`` times
    larger carry that many times the error into the exponent); the float32 bound does not move."""
    got = got.float().cpu()
    ref = ref.float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    if got.dim() == 1:
        got, ref = got[None], ref[None]
    diff = (got - ref).abs()
    if dtype == "float32":
        tol = tolerance(dtype, ref)
        STATS.append({"what": what, "dtype": dtype, "max_abs": float(diff.max()), "tol": tol})
        if float(diff.max()) > tol:
            idx = int(diff.max(dim=-1).values.argmax())
            raise AssertionError(f"{what}: max |diff| {float(diff.max()):.3e} > {tol:.3e}; first worst row {idx}; "
                                 f"rows over tolerance: {(diff.max(dim=-1).values > tol).nonzero().flatten().tolist()[:20]}")
        return
    rel = (got - ref).norm(dim=-1) / ref.norm(dim=-1).clamp_min(1e-6)
    scale = max(float(ref.abs().max()), 1.0)
    chosen = got.argmax(-1)
    lost = ref.max(-1).values - ref.gather(-1, chosen[:, None])[:, 0]        # how much worse the chosen token is, in plain logits
    STATS.append({"what": what, "dtype": dtype, "rows": int(rel.numel()), "row_max": float(rel.max()),
                  "row_mean": float(rel.mean()), "argmax_agree": float((chosen == ref.argmax(-1)).float().mean()),
                  "worst_choice": float(lost.max()) / scale})
    row_max, row_mean = BF16_ROW_MAX * noise, BF16_ROW_MEAN * noise
    bad = (rel > row_max).nonzero().flatten().tolist()
    assert not bad, (f"{what}: relative error of row {bad[0]} is {float(rel[bad[0]]):.3e} > {row_max:.1e} "
                     f"(rows over the bound: {bad[:20]}; mean over rows {float(rel.mean()):.3e})")
    if rel.numel() >= 8:
        assert float(rel.mean()) <= row_mean, f"{what}: mean relative row error {float(rel.mean()):.3e} > {row_mean:.1e}"
    far = (lost > BF16_NEAR_TIE * noise * scale).nonzero().flatten().tolist()
    assert not far, (f"{what}: row {far[0]} chooses a token whose plain logit is {float(lost[far[0]]):.3e} below the best "
                     f"(no near tie); rows: {far[:20]}")


# --------------------------------------------------------------------- replay traces
def round64(n: int) -> int:
    return -(-n // 64) * 64


class TraceBuilder:
    """Builds steps for ``bin/trace_run`` and remembers which (request, position)
    each output row is, and the most tokens (rounded per request to 64) live at once."""

    def __init__(self):
        self.steps: list[dict] = []
        self.rows: dict[int, list[tuple[str, int]]] = {}
        self.held: dict[str, int] = {}
        self.max_tokens = 0

    def step(self, entries: list[tuple[str, list[int], int]], end: list[str] = ()):
        """entries: (request id, tokens, position of the first of them); every position is wanted."""
        n = len(self.steps)
        rec = {"step": n, "entries": [], "end": list(end)}
        rows = []
        for rid, toks, start in entries:
            assert self.held.get(rid, 0) == start, (rid, self.held.get(rid, 0), start)
            rec["entries"].append({"id": rid, "tokens": toks, "want": list(range(len(toks)))})
            rows += [(rid, start + i) for i in range(len(toks))]
            self.held[rid] = start + len(toks)
        self.max_tokens = max(self.max_tokens, sum(round64(v) for v in self.held.values()))
        for rid in end:
            self.held.pop(rid)
        self.steps.append(rec)
        self.rows[n] = rows


def run_trace(model_dir, dtype: str, trace: TraceBuilder, out_dir, vocab: int, page_size: int = 16) -> dict:
    """Run ``bin/trace_run`` as a user would and return ``{(request, position): logits}``."""
    import json as _json
    import os
    import subprocess
    import sys

    import numpy as np

    root = Path(__file__).resolve().parent.parent
    text = "".join(_json.dumps(s) + "\n" for s in trace.steps)
    proc = subprocess.run(
        [sys.executable, str(root / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out",
         str(out_dir), "--max-tokens", str(trace.max_tokens), "--page-size", str(page_size), "--poison-free-pages"],
        input=text, capture_output=True, text=True, timeout=600, env=dict(os.environ))
    assert proc.returncode == 0, f"trace_run failed:\n{proc.stderr[-3000:]}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(trace.steps))], proc.stdout[-2000:]
    out = {}
    for n, rows in trace.rows.items():
        data = np.fromfile(Path(out_dir) / f"{n}.f32", dtype="<f4").reshape(len(rows), vocab)
        for i, key in enumerate(rows):
            assert key not in out
            out[key] = torch.from_numpy(data[i].copy())
    return out
