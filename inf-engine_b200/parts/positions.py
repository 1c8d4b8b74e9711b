"""Position encodings.

``rotary``: tables of cos and sin of ``position * inv_freq`` with
``inv_freq[i] = theta^(-2i/head_dim)`` (engine/layers.py:57-79), applied to the
pairs (i, i + head_dim/2) of q and k (:82-115).  The optional llama3 frequency
scaling is not in the reference: wavelengths below ``orig/high_freq_factor``
are kept, above ``orig/low_freq_factor`` divided by ``factor``, and blended
linearly in ``orig/wavelength`` between.  Angles and tables are float32, built
once per distinct spec and shared by the layers that use it.
"""

from __future__ import annotations

import math

import torch

from .registry import register_position


def rotary_inv_freq(spec) -> torch.Tensor:
    hd = spec.head_dim
    inv_freq = 1.0 / (spec.theta ** (torch.arange(0, hd, 2).float() / hd))
    s = spec.scaling
    if s is not None:
        if s.rope_type != "llama3":
            raise ValueError(f"rope scaling {s.rope_type!r} is not built")
        f = inv_freq.double()
        orig = float(s.original_max_position_embeddings)
        wavelen = 2.0 * math.pi / f
        smooth = (orig / wavelen - s.low_freq_factor) / (s.high_freq_factor - s.low_freq_factor)
        blended = (1.0 - smooth) * f / s.factor + smooth * f
        out = torch.where(wavelen < orig / s.high_freq_factor, f,
                          torch.where(wavelen > orig / s.low_freq_factor, f / s.factor, blended))
        inv_freq = out.float()
    return inv_freq


def rotary_tables(spec) -> tuple[torch.Tensor, torch.Tensor]:
    """cos, sin: float32 [max_positions, head_dim/2] on the CPU."""
    inv_freq = rotary_inv_freq(spec)
    angles = torch.outer(torch.arange(spec.max_positions).float(), inv_freq)
    return angles.cos().contiguous(), angles.sin().contiguous()


@register_position("none")
class NoPosition:
    @staticmethod
    def expected_tensors(spec):
        return {}

    def __init__(self, spec, tensors, rt):
        self.spec = spec

    def rotary_tables(self):
        return None

    def rotate(self, q, k, ctx):
        return None


@register_position("rotary")
class Rotary:
    @staticmethod
    def expected_tensors(spec):
        return {}

    def __init__(self, spec, tensors, rt):
        if spec.head_dim % 2:
            raise ValueError("rotary embeddings need an even head_dim")
        self.spec = spec
        key = ("rotary", spec)
        if key not in rt.shared:
            cos, sin = rotary_tables(spec)
            rt.shared[key] = (cos.to(rt.device), sin.to(rt.device))
        self.cos, self.sin = rt.shared[key]

    def rotary_tables(self):
        return self.cos, self.sin

    def rotate(self, q, k, ctx):
        return None
