"""``y = x W^T`` with the weight in the checkpoint's (out, in) layout
(engine/layers.py:48-50).

Which kernel runs is decided by the dtypes:
  * float32 activations, or a weight kept in float32: the CUDA-core kernel of
    this package (float32 products and sums, no tensor cores);
  * bfloat16 activations and weight: the library matrix product (cuBLAS through
    ``torch.mm``), which is what the reference's engine uses for every
    projection, or this package's own kernels where they are registered for the
    shape.
"""

from __future__ import annotations

import torch

from .. import kernels


class Linear:
    def __init__(self, weight: torch.Tensor, rt, name: str = "linear"):
        assert weight.dim() == 2 and weight.is_contiguous()
        self.weight = weight
        self.rt = rt
        self.name = name
        self.out_features, self.in_features = weight.shape

    def streams(self, n_rows: int, normed: bool = False) -> bool:
        """True when the weight-streaming kernel of this package takes this product:
        bfloat16 weight and activations, few rows, K a multiple of 8.  ``normed``: the product is to
        carry a norm in its prologue.  A weight of real size (four million elements and more) is
        streamed only by the kernel with the shared-memory ring: the other one, for the widths of tiny
        models, reads such a weight at a fraction of the HBM rate.  The ring kernel wants K a multiple
        of 256 and keeps the rows of a normed input in shared memory; where it does not take the
        product (9 to 16 rows of more than 3,072 columns, say) the library product stands in."""
        if not (self.weight.dtype is torch.bfloat16 and self.rt.act_dtype is torch.bfloat16
                and 0 < n_rows <= kernels.STREAM_BEST_ROWS and self.in_features % 8 == 0):
            return False
        if self.out_features * self.in_features >= (1 << 22):
            return kernels.gemm_stream_ring_supports(n_rows, self.out_features, self.in_features, normed)
        return True

    def stream(self, x: torch.Tensor, out: torch.Tensor, n_rows: int, epi: str = "bf16", gain=None, eps: float = 0.0,
               row_index=None) -> torch.Tensor:
        """The product through the weight-streaming kernel, with its fused prologue and epilogue."""
        kernels.gemm_stream(x, self.weight, out, n_rows, epi, gain, eps, row_index)
        return out

    def __call__(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """Write ``x @ W^T`` into ``out`` ([M, out_features], may be a column slice)."""
        w = self.weight
        assert x.shape[1] == self.in_features and out.shape == (x.shape[0], self.out_features)
        if x.shape[0] == 0:
            return out
        if x.dtype is torch.float32 or w.dtype is torch.float32:
            kernels.gemm_simt(x, w, out)
            return out
        # bfloat16 x bfloat16
        if self.streams(x.shape[0]) and out.dtype in (torch.bfloat16, torch.float32):
            return self.stream(x, out, x.shape[0], "bf16" if out.dtype is torch.bfloat16 else "f32")
        if out.dtype is torch.bfloat16 and out.is_contiguous():
            torch.mm(x, w.t(), out=out)
        elif out.dtype is torch.float32 and out.is_contiguous():
            _mm_f32_out(x, w, out)
        else:
            kernels.gemm_simt(x, w, out)
        return out


_F32_OUT_OK: bool | None = None


def _mm_f32_out(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """bfloat16 operands, float32 result (the logits) from the library product."""
    global _F32_OUT_OK
    if _F32_OUT_OK is None:
        try:
            torch.mm(x[:1], w[:8].t(), out_dtype=torch.float32)
            _F32_OUT_OK = True
        except (TypeError, RuntimeError):
            _F32_OUT_OK = False
    if _F32_OUT_OK:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        kernels.gemm_simt(x, w, out)


# ------------------------------------------------------------------ a norm handed over between two products
# In a decode step a product that adds into the residual stream (the mixer's output projection, the feed-forward's
# second product) is followed by a product of the NORMALISED residual (gate/up, the next block's qkv, the head).
# The first can prepare the second's input while the new residual values pass through its hands: bfloat16(residual
# * gain of the norm that comes next) and the sums of squares of the rows.  The second then reads 32 KB of bfloat16
# instead of the float32 rows and the gain, and spends no time on the norm.  ``ctx.upcoming_norm`` (set by whoever
# knows the order: the block, the model) names the norm that comes next; ``ctx.handover`` carries what was prepared
# and is used only by a product whose norm is that very one.
class NormHandover:
    def __init__(self, gain, eps, xg, ssq):
        self.gain, self.eps, self.xg, self.ssq = gain, eps, xg, ssq


def stream_into_residual(linear: Linear, x: torch.Tensor, residual: torch.Tensor, n: int, ctx, rt) -> None:
    """residual += x W^T through the streaming kernel; prepares the handover for ``ctx.upcoming_norm`` if it can."""
    nxt = getattr(ctx, "upcoming_norm", None)
    ctx.handover = None
    if (nxt is not None and hasattr(nxt, "fusable_rms") and n <= 16 and linear.out_features == residual.shape[1]
            and residual.is_contiguous()):
        gain, eps = nxt.fusable_rms()
        if gain.dtype in (torch.bfloat16, torch.float32) and linear.out_features % 256 == 0:
            xg = rt.ws.take("handover_xg", (n, residual.shape[1]), torch.bfloat16)
            ssq = rt.ws.take("handover_ssq", (kernels.SSQ_SLOT, kernels.sm_count()), torch.float32)
            kernels.gemm_stream(x, linear.weight, residual, n, "residual", normout=(xg, gain, ssq))
            ctx.handover = NormHandover(gain, eps, xg, ssq)
            return
    linear.stream(x, residual, n, "residual")


def stream_normed(linear: Linear, residual: torch.Tensor, out: torch.Tensor, n: int, epi: str, norm, ctx) -> torch.Tensor:
    """out = epilogue(norm(residual) W^T) through the streaming kernel: from a handover prepared for this very norm
    (all rows, in order), else with the RMSNorm prologue."""
    gain, eps = norm.fusable_rms()
    h = getattr(ctx, "handover", None)
    ctx.handover = None
    if (h is not None and h.gain is gain and h.eps == eps and h.xg.shape[0] == n
            and kernels.stream_library().ie_gemm_stream_tma_supports(n, linear.out_features, linear.in_features, 2)):
        kernels.gemm_stream(h.xg, linear.weight, out, n, epi, eps=eps, prenormed=(h.xg, h.ssq))
        return out
    return linear.stream(residual, out, n, epi, gain, eps)

