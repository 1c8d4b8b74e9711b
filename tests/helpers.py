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
TINY = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_d": TINY_D, "tiny_e": TINY_E}
SEEDS = {"tiny_a": 0, "tiny_b": 1, "tiny_c": 2, "tiny_d": 3, "tiny_e": 4}


def make_model_dir(tmp: Path, name: str, store_dtype: str = "bfloat16", std: float = 0.05) -> Path:
    """Write a random model folder with the package's random-weights mode."""
    from inf_engine_b200.config import parse_config_dict
    from inf_engine_b200.weights import write_random_model

    cfg = parse_config_dict(TINY[name])
    out = Path(tmp) / f"{name}_{store_dtype}"
    if not (out / "model.safetensors").is_file():
        write_random_model(cfg, SEEDS[name], out, store_dtype=store_dtype, std=std)
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


def tolerance(dtype: str, ref: torch.Tensor) -> float:
    """Largest absolute logit difference allowed against the plain implementation.

    float32: summation order only.  bfloat16: activations and cache are rounded to
    8 bits of mantissa at every stage; the bound is relative to the largest logit.
    """
    scale = float(ref.abs().max())
    return (2e-5 if dtype == "float32" else 4e-2) * max(scale, 1.0)


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "") -> None:
    got = got.float().cpu()
    ref = ref.float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    diff = (got - ref).abs()
    tol = tolerance(dtype, ref)
    if float(diff.max()) > tol:
        idx = int(diff.max(dim=-1).values.argmax()) if diff.dim() > 1 else 0
        raise AssertionError(f"{what}: max |diff| {float(diff.max()):.3e} > {tol:.3e}; first worst row {idx}; "
                             f"rows over tolerance: {(diff.max(dim=-1).values > tol).nonzero().flatten().tolist()[:20]}")


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
         str(out_dir), "--max-tokens", str(trace.max_tokens), "--page-size", str(page_size)],
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
