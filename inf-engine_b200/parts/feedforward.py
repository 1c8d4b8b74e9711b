"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))`` (engine/llama_mlp.py:30-33).

Gate and up are one matrix product over the row-concatenated weights
[2*intermediate, hidden]; the activation and the product by ``up`` are one
kernel in float32 arithmetic.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import ExpectedTensor
from .linear import Linear, stream_into_residual, stream_normed
from .registry import register_feedforward


@register_feedforward("gated_mlp")
class GatedMLP:
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        return {
            spec.gate_proj: ExpectedTensor((spec.intermediate, spec.hidden)),
            spec.up_proj: ExpectedTensor((spec.intermediate, spec.hidden)),
            spec.down_proj: ExpectedTensor((spec.hidden, spec.intermediate)),
        }

    def __init__(self, spec, tensors, rt):
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not built")
        self.spec = spec
        self.rt = rt
        gate, up = tensors[spec.gate_proj], tensors[spec.up_proj]
        dtype = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
        # rows alternate gate_j, up_j: one thread of a product's epilogue then holds both halves of a pair
        both = torch.stack([gate.to(dtype), up.to(dtype)], dim=1).reshape(2 * spec.intermediate, spec.hidden)
        self.gate_up = Linear(both.contiguous(), rt, "gate_up")
        self.down = Linear(tensors[spec.down_proj], rt, "down")

    def can_fuse(self, n_tokens: int, norm) -> bool:
        return (hasattr(norm, "fusable_rms") and self.gate_up.streams(n_tokens, normed=True)
                and self.down.streams(n_tokens))

    def forward_fused(self, residual: torch.Tensor, norm, ctx) -> None:
        """residual += down(silu(gate(n)) * up(n)) with n = norm(residual), in two launches: the norm rides in
        the first product's prologue, the activation in its epilogue, the sum in the second's epilogue."""
        n = residual.shape[0]
        s, ws = self.spec, self.rt.ws
        h = ws.take("ff_hidden", (n, s.intermediate), torch.bfloat16)
        stream_normed(self.gate_up, residual, h, n, "silu_mul", norm, ctx)
        stream_into_residual(self.down, h, residual, n, ctx, self.rt)

    TCGEN05_MIN_ROWS = 128     # below one tile of rows the library product is the better choice

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        n = x.shape[0]
        s, ws, dt = self.spec, self.rt.ws, self.rt.act_dtype
        h = ws.take("ff_hidden", (n, s.intermediate), dt)
        w = self.gate_up.weight
        if (dt is torch.bfloat16 and w.dtype is torch.bfloat16 and n >= self.TCGEN05_MIN_ROWS
                and kernels.gemm_tcgen05_supports(n, 2 * s.intermediate, s.hidden, x.stride(0), w.stride(0))):
            # gate/up on the tcgen05 tensor cores with silu(gate)*up in the epilogue: the [n, 2*intermediate]
            # matrix never goes to memory
            kernels.gemm_tcgen05(x, w, h, "silu_mul")
        else:
            gu = self.gate_up(x, ws.take("ff_gate_up", (n, 2 * s.intermediate), dt))
            kernels.silu_mul(gu, h, interleaved=True)
        return self.down(h, ws.take("ff_out", (n, s.hidden), dt))
