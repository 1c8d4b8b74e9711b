"""Plain, slow, whole-sequence implementation of the dense Llama decoder.

This file is the oracle of the test-suite.  It is written from the formulas of
the reference project (waleedalfar/inf-engine, paths below are relative to that
project's root) and shares no code with the product package: it takes the
``config.json`` dictionary itself and a ``{tensor name: float32 tensor}``
dictionary, keeps no cache, and recomputes every position of a sequence on the
CPU in float32.

The comparison ``tests/golden/make_golden.py`` ran this file against the
reference's own ``LlamaModel.forward`` on tiny random models on the CPU; the
small outputs it wrote are committed under ``tests/golden/``.  The llama3
frequency scaling has no counterpart in the reference and rests on its formula
alone.
"""

from __future__ import annotations

import math

import torch


# --------------------------------------------------------------------------- norms
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps) * weight`` — engine/layers.py:11-25."""
    rms = torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (x / rms) * weight


# ------------------------------------------------------------------ position encoding
def rope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    """``1 / theta^(2i/head_dim)`` for i in [0, head_dim/2) — engine/layers.py:72-74."""
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))


def llama3_scale_inv_freq(inv_freq: torch.Tensor, scaling: dict) -> torch.Tensor:
    """llama3 frequency scaling (no counterpart in the reference; formula only).

    Wavelengths shorter than ``orig/high_freq_factor`` are kept, longer than
    ``orig/low_freq_factor`` are divided by ``factor``, and the band between is
    blended linearly in ``orig/wavelength``.
    """
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    low_wavelen = orig / low
    high_wavelen = orig / high
    out = []
    for f in inv_freq.tolist():
        wavelen = 2.0 * math.pi / f
        if wavelen < high_wavelen:
            out.append(f)
        elif wavelen > low_wavelen:
            out.append(f / factor)
        else:
            smooth = (orig / wavelen - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return torch.tensor(out, dtype=torch.float32)


def rope_tables(config: dict, n_positions: int) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables of shape (n_positions, head_dim) — engine/layers.py:57-79."""
    hd = head_dim_of(config)
    inv_freq = rope_inv_freq(hd, float(config.get("rope_theta", 10000.0)))
    scaling = config.get("rope_scaling")
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind == "llama3":
            inv_freq = llama3_scale_inv_freq(inv_freq, scaling)
        elif kind not in (None, "default"):
            raise ValueError(f"plain implementation knows no rope scaling {kind!r}")
    positions = torch.arange(n_positions).float()
    angles = torch.outer(positions, inv_freq)
    cos = torch.cat([angles.cos(), angles.cos()], dim=-1)
    sin = torch.cat([angles.sin(), angles.sin()], dim=-1)
    return cos, sin


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """``[-x2, x1]`` for ``x = [x1, x2]`` split on the last axis — engine/layers.py:82-85."""
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x*cos + rotate_half(x)*sin``; x is (heads, T, hd), tables (T, hd) — engine/layers.py:107-115."""
    return x * cos[None] + rotate_half(x) * sin[None]


# ------------------------------------------------------------------------- attention
def head_dim_of(config: dict) -> int:
    """``head_dim`` key if present, else hidden/heads — engine/config.py:60-66."""
    hd = config.get("head_dim")
    if hd:
        return int(hd)
    return int(config["hidden_size"]) // int(config["num_attention_heads"])


def attention(
    h: torch.Tensor,
    wq: torch.Tensor,
    wk: torch.Tensor,
    wv: torch.Tensor,
    wo: torch.Tensor,
    config: dict,
    cos: torch.Tensor,
    sin: torch.Tensor,
    window: int | None = None,
) -> torch.Tensor:
    """Causal grouped-query self-attention over a whole sequence.

    h is (T, hidden).  Projections ``x @ W.T`` (engine/llama_attention.py:83-85),
    head split (:88-90), rotation of q and k (:98), kv head c serving query heads
    c*g .. c*g+g-1 (:27-44), scores scaled by head_dim**-0.5 with the causal rule
    "key j visible to query i iff j <= i" (:109-137), heads merged head-major and
    projected by W_o (:140-141).  ``window`` (not in the reference) limits a query
    to the last ``window`` keys, itself included.
    """
    T = h.shape[0]
    n_head = int(config["num_attention_heads"])
    n_kv = int(config.get("num_key_value_heads", n_head))
    hd = head_dim_of(config)
    group = n_head // n_kv
    q = (h @ wq.T).view(T, n_head, hd).transpose(0, 1)  # (H, T, hd)
    k = (h @ wk.T).view(T, n_kv, hd).transpose(0, 1)
    v = (h @ wv.T).view(T, n_kv, hd).transpose(0, 1)
    q = apply_rope(q, cos[:T], sin[:T])
    k = apply_rope(k, cos[:T], sin[:T])
    k = k[:, None].expand(n_kv, group, T, hd).reshape(n_head, T, hd)
    v = v[:, None].expand(n_kv, group, T, hd).reshape(n_head, T, hd)
    scores = (q @ k.transpose(1, 2)) * (hd ** -0.5)  # (H, T, T)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    allowed = j <= i
    if window is not None:
        allowed = allowed & (j > i - window)
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = probs @ v  # (H, T, hd)
    out = out.transpose(0, 1).reshape(T, n_head * hd)
    return out @ wo.T


# ---------------------------------------------------------------------- feed-forward
def silu(x: torch.Tensor) -> torch.Tensor:
    """``x * sigmoid(x)`` — engine/layers.py:28-30."""
    return x * torch.sigmoid(x)


def swiglu(h: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """``down(silu(gate(x)) * up(x))`` — engine/llama_mlp.py:30-33."""
    return (silu(h @ wg.T) * (h @ wu.T)) @ wd.T


# ----------------------------------------------------------------------------- block
def block(x: torch.Tensor, w: dict, prefix: str, config: dict, cos, sin) -> torch.Tensor:
    """Pre-norm residual block — engine/llama_block.py:50-62."""
    eps = float(config.get("rms_norm_eps", 1e-5))
    h = rms_norm(x, w[prefix + "input_layernorm.weight"], eps)
    x = x + attention(
        h,
        w[prefix + "self_attn.q_proj.weight"],
        w[prefix + "self_attn.k_proj.weight"],
        w[prefix + "self_attn.v_proj.weight"],
        w[prefix + "self_attn.o_proj.weight"],
        config,
        cos,
        sin,
    )
    h = rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps)
    x = x + swiglu(
        h,
        w[prefix + "mlp.gate_proj.weight"],
        w[prefix + "mlp.up_proj.weight"],
        w[prefix + "mlp.down_proj.weight"],
    )
    return x


# ----------------------------------------------------------------------------- model
def forward_logits(weights: dict, config: dict, token_ids: list[int], rows: list[int] | None = None) -> torch.Tensor:
    """Logits (T, vocab) of one whole sequence — engine/llama_model.py:128-149; with ``rows`` only
    those positions go through the final norm and the head (a large vocabulary is slow on the CPU).

    Embedding row gather without scaling (:128), the blocks in order (:139-144),
    final norm (:147) and the head, which is the embedding table when
    ``tie_word_embeddings`` is set or ``lm_head.weight`` is absent
    (engine/llama_weights.py:39-47).
    """
    w = {k: v.float() for k, v in weights.items()}
    ids = torch.tensor(token_ids, dtype=torch.long)
    x = w["model.embed_tokens.weight"][ids]
    cos, sin = rope_tables(config, len(token_ids))
    for i in range(int(config["num_hidden_layers"])):
        x = block(x, w, f"model.layers.{i}.", config, cos, sin)
    if rows is not None:
        x = x[torch.tensor(rows, dtype=torch.long)]
    x = rms_norm(x, w["model.norm.weight"], float(config.get("rms_norm_eps", 1e-5)))
    if config.get("tie_word_embeddings", False) or "lm_head.weight" not in w:
        head = w["model.embed_tokens.weight"]
    else:
        head = w["lm_head.weight"]
    return x @ head.T


def greedy_generate(weights: dict, config: dict, prompt: list[int], n_new: int) -> list[int]:
    """Cache-free greedy continuation — engine/llama_model.py:152-175."""
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(forward_logits(weights, config, ids)[-1].argmax()))
    return ids[len(prompt):]


# -------------------------------------------------------------------------- sampling
def apply_repetition_penalty(logits: torch.Tensor, context: list[int], penalty: float, window: int = 256) -> torch.Tensor:
    """Flat penalty on the unique tokens of the last ``window`` context tokens:
    positive logits divided, negative multiplied — engine/sampling.py:90-135."""
    out = logits.clone()
    for t in set(context[-window:]):
        out[t] = out[t] * penalty if out[t] < 0 else out[t] / penalty
    return out


def top_k_filter(logits: torch.Tensor, k: int) -> torch.Tensor:
    """Keep logits >= the k-th largest (ties kept), k clamped to [1, V] — engine/sampling.py:138-153."""
    k = max(1, min(k, logits.numel()))
    kth = torch.topk(logits, k).values[-1]
    return logits.masked_fill(logits < kth, float("-inf"))


def top_p_filter(logits: torch.Tensor, p: float) -> torch.Tensor:
    """Drop a token when the probability mass before it (descending order) is
    already >= p; the most likely token always stays — engine/sampling.py:156-177."""
    sorted_logits, sorted_idx = torch.sort(logits, descending=True)
    probs = torch.softmax(sorted_logits, dim=-1)
    before = probs.cumsum(dim=-1) - probs
    drop_sorted = before >= p
    drop_sorted[0] = False
    drop = torch.zeros_like(drop_sorted).scatter(0, sorted_idx, drop_sorted)
    return logits.masked_fill(drop, float("-inf"))


def filtered_distribution(
    logits: torch.Tensor,
    mode: str,
    temperature: float = 1.0,
    top_k: int = 50,
    top_p: float = 0.9,
) -> torch.Tensor:
    """Probabilities the next token is drawn from — engine/sampling.py:72-86.

    greedy: one-hot at the argmax.  Otherwise logits/temperature, the mode's
    filter, softmax.  ``temperature`` mode is the unfiltered softmax.
    """
    logits = logits.float()
    if mode == "greedy":
        out = torch.zeros_like(logits)
        out[int(logits.argmax())] = 1.0
        return out
    scaled = logits / temperature
    if mode == "top_k":
        scaled = top_k_filter(scaled, top_k)
    elif mode == "top_p":
        scaled = top_p_filter(scaled, top_p)
    elif mode != "temperature":
        raise ValueError(mode)
    return torch.softmax(scaled, dim=-1)
