"""RMSNorm: ``x / sqrt(mean(x^2) + eps) * gain`` (engine/layers.py:11-25), with
float32 statistics whatever the activation dtype, fused with the residual sum
that precedes it in a pre-norm block (engine/llama_block.py:53-62)."""

from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import ExpectedTensor
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm:
    @staticmethod
    def expected_tensors(spec):
        return {spec.weight: ExpectedTensor((spec.size,), init="gain")}

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.rt = rt
        self.gain = tensors[spec.weight]
        self.eps = float(spec.eps)
        self.size = spec.size

    def fusable_rms(self):
        """(gain, eps) for kernels that apply this norm inside a matrix product's prologue."""
        return self.gain, self.eps

    def add_norm(self, residual: torch.Tensor, delta: torch.Tensor | None, out_name: str = "normed") -> torch.Tensor:
        out = self.rt.ws.take(out_name, tuple(residual.shape), self.rt.act_dtype)
        kernels.rmsnorm(residual, delta, self.gain, out, self.eps)
        return out

    def gather_norm(self, residual: torch.Tensor, delta: torch.Tensor | None, row_index: torch.Tensor,
                    n_rows: int, out_name: str = "normed_rows") -> torch.Tensor:
        out = self.rt.ws.take(out_name, (n_rows, self.size), self.rt.act_dtype)
        kernels.rmsnorm(residual, delta, self.gain, out, self.eps, row_index=row_index)
        return out
