"""Load a checkpoint by tensor name against what the model's parts expect.

Every part of a model declares the tensors it needs with their shapes
(``parts.registry.expected_tensors``).  The loader compares that table with the
checkpoint and raises ONE error that lists every missing tensor, every
unexpected one and every wrong shape.  The reference checks only two names and
no shape (engine/llama_weights.py:146-149), so a bad checkpoint surfaces there
as a ``KeyError`` in the middle of a forward pass.

Precision of what is kept on the device:
  * run dtype float32: every floating tensor becomes float32;
  * run dtype bfloat16: 16-bit tensors become bfloat16, a tensor stored in 32-bit
    (or 64-bit) floating point stays float32 — kernels take either;
  * integer tensors become int32.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import torch

from .safetensors_io import StoredTensor, open_checkpoint


@dataclass(frozen=True)
class ExpectedTensor:
    """What a part says about a tensor it reads: its shape, and how the random-weights mode should draw it
    (``"normal"``: N(0, std), matrices, biases, learned vectors; ``"gain"``: 1 + U(-spread, spread), a norm's
    multiplier)."""

    shape: tuple[int, ...]
    init: str = "normal"


class WeightsError(ValueError):
    """The checkpoint does not match the model; lists everything that is wrong."""

    def __init__(self, missing, unexpected, wrong_shape, where=""):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        lines = [f"checkpoint {where} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {tuple(e)}, found {tuple(f)}" for n, e, f in self.wrong_shape))
        super().__init__("\n".join(lines))


def kept_dtype(stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor has on the device (see the module docstring)."""
    if not stored.is_floating_point:
        return torch.int32
    if run_dtype is torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


# Buffers that older checkpoints of this family store beside their weights and that no model reads (the rotary
# frequencies are computed from the configuration).  They are passed over; every other unknown name is an error.
IGNORED_SUFFIXES = (".rotary_emb.inv_freq",)


def ignored_buffers(found) -> list[str]:
    return sorted(n for n in found if n.endswith(IGNORED_SUFFIXES))


def check_names_and_shapes(found: dict[str, tuple[int, ...]], expected: dict[str, ExpectedTensor],
                           optional: tuple[str, ...] = (), where: str = "") -> None:
    missing = [n for n in expected if n not in found]
    unexpected = [n for n in found if n not in expected and n not in optional and not n.endswith(IGNORED_SUFFIXES)]
    wrong = [(n, expected[n].shape, found[n]) for n in expected if n in found and tuple(found[n]) != tuple(expected[n].shape)]
    if missing or unexpected or wrong:
        raise WeightsError(missing, unexpected, wrong, where)


def load_weights(model_dir: str | Path, expected: dict[str, ExpectedTensor], run_dtype: torch.dtype,
                 device: str | torch.device, optional: tuple[str, ...] = ()) -> dict[str, torch.Tensor]:
    """Tensors of ``model_dir`` on ``device``, validated against ``expected``."""
    stored: dict[str, StoredTensor] = open_checkpoint(model_dir)
    check_names_and_shapes({n: s.shape for n, s in stored.items()}, expected, optional, where=str(model_dir))
    passed_over = ignored_buffers(stored)
    if passed_over:
        import warnings
        warnings.warn(f"checkpoint {model_dir}: {len(passed_over)} stored buffers are not weights and were passed over "
                      f"({passed_over[0]}, ...)", stacklevel=2)
    out: dict[str, torch.Tensor] = {}
    for name in expected:
        t = stored[name].read()
        out[name] = t.to(device=device, dtype=kept_dtype(t.dtype, run_dtype)).contiguous()
    return out
