"""The pre-norm residual block: ``x += mixer(norm(x)); x += ff(norm(x))``
(engine/llama_block.py:50-62).  The sums are folded into the norm that follows
them: a block hands on the residual and a delta that is not added yet."""

from __future__ import annotations

from .. import kernels
from .registry import (
    build_feedforward,
    build_mixer,
    build_norm,
    feedforward_class,
    mixer_class,
    norm_class,
    register_block,
)


@register_block("prenorm")
class PreNormBlock:
    @staticmethod
    def expected_tensors(spec):
        out = {}
        out.update(norm_class(spec.mixer_norm).expected_tensors(spec.mixer_norm))
        out.update(mixer_class(spec.mixer).expected_tensors(spec.mixer))
        out.update(norm_class(spec.ff_norm).expected_tensors(spec.ff_norm))
        out.update(feedforward_class(spec.feedforward).expected_tensors(spec.feedforward))
        return out

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.mixer_norm = build_norm(spec.mixer_norm, tensors, rt)
        self.mixer = build_mixer(spec.mixer, tensors, rt)
        self.ff_norm = build_norm(spec.ff_norm, tensors, rt)
        self.feedforward = build_feedforward(spec.feedforward, tensors, rt)

    @property
    def graph_safe(self) -> bool:
        """Whether a step through this block may be captured as a CUDA graph: every part says that it reads the
        batch's numbers on the device only and never waits for the device (a part that says nothing does not)."""
        return all(getattr(p, "graph_safe", False) for p in (self.mixer, self.feedforward))

    def forward(self, residual, pending, ctx, cache):
        n = ctx.n_tokens
        # a part may offer forward_fused(residual, norm, ...): it applies the norm and adds its own
        # result into the residual inside its kernels (worth it for the few rows of a decode step)
        # ctx.upcoming_norm tells a fused part which norm follows its product into the residual (it may prepare
        # that norm's input); ctx.handover is what the part before prepared, void as soon as the residual changes
        after_block = getattr(ctx, "norm_after_block", None)
        ff_fuses = _fuses(self.feedforward, n, self.ff_norm)
        if _fuses(self.mixer, n, self.mixer_norm):
            if pending is not None:
                kernels.residual_add(residual, pending)
                ctx.handover = None
            ctx.upcoming_norm = self.ff_norm if ff_fuses else None
            self.mixer.forward_fused(residual, self.mixer_norm, ctx, cache)
            a = None
        else:
            ctx.handover = None
            h = self.mixer_norm.add_norm(residual, pending)
            a = self.mixer.forward(h, ctx, cache)
        if ff_fuses:
            if a is not None:
                kernels.residual_add(residual, a)
                ctx.handover = None
            ctx.upcoming_norm = after_block
            self.feedforward.forward_fused(residual, self.ff_norm, ctx)
            ctx.upcoming_norm = None
            return residual, None
        ctx.handover = None
        ctx.upcoming_norm = None
        h = self.ff_norm.add_norm(residual, a)
        m = self.feedforward.forward(h, ctx)
        return residual, m


def _fuses(part, n_tokens: int, norm) -> bool:
    can = getattr(part, "can_fuse", None)
    return bool(can and can(n_tokens, norm))
