"""The pre-norm residual block: ``x += mixer(norm(x)); x += ff(norm(x))``
(engine/llama_block.py:50-62).  The sums are folded into the norm that follows
them: a block hands on the residual and a delta that is not added yet."""

from __future__ import annotations

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

    def forward(self, residual, pending, ctx, cache):
        h = self.mixer_norm.add_norm(residual, pending)
        a = self.mixer.forward(h, ctx, cache)
        h = self.ff_norm.add_norm(residual, a)
        m = self.feedforward.forward(h, ctx)
        return residual, m
