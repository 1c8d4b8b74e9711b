"""Random-weights mode: write a model folder from a configuration and a seed.

The reference has no such loader mode; its tests hand-build dictionaries with
unit gains and standard deviation 1 (tests/test_paged_cache.py:42-72), which
hides faults in gains and scales.  Here matrices are N(0, std) and norm gains
1 + U(-spread, spread), drawn on the CPU from one seeded generator in the order
of the model's tensor table, so the same seed gives the same folder everywhere.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def random_tensors(expected: dict, seed: int, std: float = 0.02, gain_spread: float = 0.1,
                   store_dtype: str = "bfloat16") -> dict[str, torch.Tensor]:
    """One tensor per entry of ``expected`` (name -> ExpectedTensor), in that order.

    A tensor that its part declares as a gain (``ExpectedTensor.init == "gain"``) is 1 + U(-spread, spread);
    everything else, one-dimensional or not, is N(0, std).  Large matrices are drawn in slabs so that a
    128k-row table needs no second copy.
    """
    dtype = _STORE[store_dtype]
    g = torch.Generator().manual_seed(int(seed))
    out = {}
    for name, exp in expected.items():
        shape = tuple(exp.shape)
        if getattr(exp, "init", "normal") == "gain":
            t = 1.0 + (torch.rand(shape, generator=g) * (2 * gain_spread) - gain_spread)
            out[name] = t.to(dtype)
        elif getattr(exp, "init", "normal") != "normal":
            raise ValueError(f"tensor {name!r}: unknown random initialisation {exp.init!r}")
        else:
            t = torch.empty(shape, dtype=dtype)
            rows = shape[0]
            slab = max(1, (1 << 24) // max(1, t[0].numel()))
            for r in range(0, rows, slab):
                n = min(slab, rows - r)
                t[r:r + n] = (torch.randn((n,) + shape[1:], generator=g) * std).to(dtype)
            out[name] = t
    return out


def write_random_model(config, seed: int, out_dir: str | Path, store_dtype: str = "bfloat16",
                       std: float = 0.02, gain_spread: float = 0.1) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` under ``out_dir``."""
    from ..parts.registry import expected_tensors  # late: parts import the spec classes

    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    spec = config.model_spec()
    tensors = random_tensors(expected_tensors(spec), seed, std, gain_spread, store_dtype)
    with open(out_dir / "config.json", "w") as f:
        json.dump(config.to_hf_dict(), f, indent=1)
    write_safetensors(out_dir / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": seed, "init": f"normal({std}) gains 1+-{gain_spread}"})
    return out_dir
