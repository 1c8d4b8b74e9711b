"""Greedy, temperature, top-k and top-p sampling with the reference's option
names and meanings (engine/sampling.py:16-87), on the device.

Differences that are on purpose:
  * ``temperature`` is a mode of its own (the reference reaches it as top-p
    with p = 1);
  * the draw is the inverse CDF at a number hashed from (seed, request,
    position), so a row's token does not depend on what else is in the batch;
    the reference shares one ``torch.Generator`` across the batch (:47, :87);
  * everything is float32; the reference samples in the logits' dtype.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

import numpy as np
import torch

from .. import kernels

REPETITION_PENALTY_WINDOW = 256   # engine/sampling.py:90
_MASK64 = (1 << 64) - 1


class SamplingMode(str, Enum):
    GREEDY = "greedy"
    TEMPERATURE = "temperature"
    TOP_K = "top_k"
    TOP_P = "top_p"


@dataclass
class SamplingConfig:
    """Decoding options; names and defaults as engine/sampling.py:24-47, plus ``seed``."""

    mode: SamplingMode = SamplingMode.GREEDY
    temperature: float = 1.0
    top_k: int = 50
    top_p: float = 0.9
    repetition_penalty: float = 1.0
    seed: int = 0

    def __post_init__(self):
        self.mode = SamplingMode(self.mode)

    def validate(self) -> None:
        if self.mode is not SamplingMode.GREEDY and self.temperature <= 0.0:
            raise ValueError("temperature must be > 0 for sampling modes")   # engine/sampling.py:75-76
        if self.mode is SamplingMode.TOP_P and not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")                      # engine/sampling.py:167-168
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be positive")


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK64
    return x ^ (x >> 31)


def uniform_of(seed: int, key: int) -> float:
    """The number in [0, 1) the device draws for (seed, key): 24 bits of a hash."""
    h = splitmix64(splitmix64(seed & _MASK64) ^ (key & _MASK64))
    return (h >> 40) / 16777216.0


def request_key(request_id: int, position: int) -> int:
    """Key of a draw: which request and how many tokens it had generated."""
    return ((int(request_id) & 0xFFFFFFFF) << 32) | (int(position) & 0xFFFFFFFF)


def pack_rows(configs: list[SamplingConfig], keys: list[int], vocab: int) -> np.ndarray:
    """The sampling kernel's records, int32 [n, 7]: temperature (float bits; <= 0 is greedy),
    top_p (float bits; >= 1 is off), top_k (<= 0 is off), seed low/high, key low/high."""
    m = len(configs)
    rows = np.zeros((m, 7), dtype=np.int32)
    f = rows.view(np.float32)
    u = rows.view(np.uint32)
    for i, c in enumerate(configs):
        c.validate()
        if c.mode is SamplingMode.GREEDY:
            f[i, 0], f[i, 1], rows[i, 2] = 0.0, 1.0, 0
        else:
            f[i, 0] = c.temperature
            f[i, 1] = c.top_p if c.mode is SamplingMode.TOP_P else 1.0
            rows[i, 2] = max(1, min(int(c.top_k), vocab)) if c.mode is SamplingMode.TOP_K else 0
        seed, key = c.seed & _MASK64, keys[i] & _MASK64
        u[i, 3], u[i, 4] = seed & 0xFFFFFFFF, seed >> 32
        u[i, 5], u[i, 6] = key & 0xFFFFFFFF, key >> 32
    return rows


class Sampler:
    def __init__(self, rt):
        self.rt = rt

    def sample(self, logits: torch.Tensor, configs: list[SamplingConfig], keys: list[int],
               contexts: list[list[int]] | None = None) -> torch.Tensor:
        """One token per row of float32 ``logits`` [M, V] -> int32 [M] on the device.

        ``contexts[i]`` (tokens seen so far) matters only to rows with a repetition
        penalty; the penalty rewrites the logits in place, as the reference's does on
        a copy (engine/sampling.py:120).
        """
        m, vocab = logits.shape
        assert len(configs) == m and len(keys) == m
        out = self.rt.ws.take("sampled", (m,), torch.int32)
        pens = [c.repetition_penalty for c in configs]
        if contexts is not None and any(p != 1.0 for p in pens):
            w = REPETITION_PENALTY_WINDOW
            ctx = np.full((m, w), -1, dtype=np.int32)
            for i, c in enumerate(contexts):
                if pens[i] != 1.0 and c:
                    tail = c[-w:]
                    ctx[i, :len(tail)] = tail
            pen = np.asarray(pens, dtype=np.float32).view(np.int32)
            dev = self.rt.staging.upload(np.concatenate([ctx.reshape(-1), pen]))
            kernels.repetition_penalty(logits, dev[:m * w].view(m, w), dev[m * w:].view(torch.float32))
        if all(c.mode is SamplingMode.GREEDY for c in configs):
            kernels.argmax(logits, out)
            return out
        rows = pack_rows(configs, keys, vocab)
        dev = self.rt.staging.upload(rows.reshape(-1)).view(m, 7)
        kernels.sample(logits, dev, out)
        return out
