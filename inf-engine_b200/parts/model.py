"""A decoder put together from parts: token table, blocks run in the order of
the schedule, final norm on the rows whose logits are wanted, head
(engine/llama_model.py:128-149).  The reference computes logits for every
position (:148); here the head runs on the gathered rows only and its result
is float32."""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import CacheManager, CacheRequirement
from .attention import CacheView
from .linear import Linear, stream_normed
from ..weights.loader import ExpectedTensor
from .registry import block_class, build_block, build_norm, norm_class, register_model


@register_model("decoder")
class DecoderModel:
    @staticmethod
    def expected_tensors(spec) -> dict:
        """The token table, the layers in order, the final norm, the head."""
        out = {spec.embedding: ExpectedTensor((spec.vocab_size, spec.hidden))}
        for blk in spec.layers:
            out.update(block_class(blk).expected_tensors(blk))
        out.update(norm_class(spec.final_norm).expected_tensors(spec.final_norm))
        if spec.head is not None:
            out[spec.head] = ExpectedTensor((spec.vocab_size, spec.hidden))
        return out

    def __init__(self, spec, tensors: dict, rt):
        self.spec = spec
        self.rt = rt
        self.embedding = tensors[spec.embedding]
        self.layers = [build_block(b, tensors, rt) for b in spec.layers]
        self.final_norm = build_norm(spec.final_norm, tensors, rt)
        head = tensors[spec.head] if spec.head is not None else self.embedding   # tied: one buffer
        self.head = Linear(head, rt, "head")
        for i, e in enumerate(spec.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_from is not None and not (0 <= e.cache_from < i and spec.schedule[e.cache_from].cache_from is None):
                raise ValueError(f"schedule entry {i} must read the cache of an earlier entry that owns one")
        # a decode step is captured as a graph only if every block that runs says it may be
        self.graph_safe = all(getattr(self.layers[e.layer], "graph_safe", False) for e in spec.schedule)
        self._views: list[CacheView] | None = None

    # ------------------------------------------------------------------ cache
    def cache_requirements(self) -> list[CacheRequirement]:
        """One requirement per schedule entry; a run that reads another run's cache needs none."""
        reqs = []
        for e in self.spec.schedule:
            if e.cache_from is not None:
                reqs.append(CacheRequirement(kind="none"))
            else:
                reqs.append(self.layers[e.layer].mixer.cache_requirement())
        return reqs

    def bind_cache(self, manager: CacheManager) -> None:
        views = []
        for i, e in enumerate(self.spec.schedule):
            src = i if e.cache_from is None else e.cache_from
            b = manager.bindings[src]
            if b.kind == "kv":
                g = manager.kv_groups[b.group]
                views.append(CacheView("kv", b.group, g.k[b.row], g.v[b.row], None, write=e.cache_from is None))
            elif b.kind == "state":
                g = manager.state_groups[b.group]
                views.append(CacheView("state", b.group, None, None, g.data[b.row], write=e.cache_from is None))
            else:
                views.append(CacheView("none"))
        self._views = views

    # ---------------------------------------------------------------- forward
    def embed(self, ctx) -> torch.Tensor:
        """The float32 residual stream [n_tokens, hidden] that the first block meets."""
        residual = self.rt.ws.take("residual", (ctx.n_tokens, self.spec.hidden), torch.float32)
        kernels.embed_gather(ctx.token_ids, self.embedding, residual)
        return residual

    def finish_logits(self, logits: torch.Tensor, ctx) -> torch.Tensor:
        """What a derived top level does to the head's float32 logits (in place) before they leave; nothing here."""
        return logits

    def forward(self, ctx) -> torch.Tensor | None:
        """Run the step's tokens through every scheduled layer; float32 logits
        [n_wanted, vocab] at ``ctx.logit_rows`` (None when nothing is wanted)."""
        assert self._views is not None, "bind_cache() first"
        rt, spec = self.rt, self.spec
        n = ctx.n_tokens
        residual = self.embed(ctx)
        pending = None
        ctx.handover = None
        last = len(spec.schedule) - 1
        for i, e in enumerate(spec.schedule):
            # the norm that the residual meets after this block: the next block's first, or the final one
            nxt = self.layers[spec.schedule[i + 1].layer] if i < last else None
            ctx.norm_after_block = getattr(nxt, "mixer_norm", None) if nxt is not None else self.final_norm
            residual, pending = self.layers[e.layer].forward(residual, pending, ctx, self._views[i])
        ctx.norm_after_block = None
        m = ctx.n_logits
        if m == 0:
            return None
        return self.finish_logits(self._head_logits(residual, pending, ctx, n, m), ctx)

    def _head_logits(self, residual, pending, ctx, n: int, m: int) -> torch.Tensor:
        rt, spec = self.rt, self.spec
        logits = rt.ws.take("logits", (m, spec.vocab_size), torch.float32)
        if self.head.streams(m, normed=True) and hasattr(self.final_norm, "fusable_rms"):
            # final norm on the gathered rows inside the head product
            if pending is not None:
                kernels.residual_add(residual, pending)
                ctx.handover = None
            if m == n and getattr(ctx, "handover", None) is not None:
                # every row is wanted (a decode step): the last block may have prepared the final norm's input
                return stream_normed(self.head, residual, logits, m, "f32", self.final_norm, ctx)
            gain, eps = self.final_norm.fusable_rms()
            return self.head.stream(residual, logits, m, "f32", gain, eps, row_index=ctx.logit_rows)
        h = self.final_norm.gather_norm(residual, pending, ctx.logit_rows, m)
        return self.head(h, logits)
