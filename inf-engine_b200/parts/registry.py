"""Registries from a spec's ``kind`` to the class that runs it.

Interfaces (``rt`` is the Runtime, ``tensors`` the loaded checkpoint by name,
``ctx`` the StepContext of the step):

Norm            expected_tensors(spec) -> {name: ExpectedTensor}
                __init__(spec, tensors, rt)
                add_norm(residual, delta, out_name="normed") -> normed
                    residual (float32 [N, d]) takes ``+= delta`` (delta may be None) and the
                    normalised rows come back in the activation dtype
                gather_norm(residual, delta, row_index, n_rows) -> normed rows [n_rows, d]
PositionEncoding expected_tensors(spec); __init__(spec, tensors, rt)
                rotary_tables() -> (cos, sin) float32 [max_positions, head_dim/2] or None
                rotate(q, k, ctx) for encodings that are not table rotations (default: nothing)
                score_bias() -> float32 [n_heads, D] or None (optional): added to the score of a key that lies
                    d positions back as bias[head, min(d, D - 1)]; the attention mixer then runs its general kernel
Mixer           expected_tensors(spec); __init__(spec, tensors, rt)
                cache_requirement() -> CacheRequirement   (pages of keys/values, a state, or none)
                forward(x, ctx, cache) -> [N, hidden] in the activation dtype
                    cache is a CacheView: the pools or the state of this run, and whether to write
                graph_safe: bool   (True when forward reads batch metadata on the device only)
FeedForward     expected_tensors(spec); __init__(spec, tensors, rt); forward(x, ctx) -> [N, hidden]
                graph_safe: bool   (as for a mixer; a part that does not say so keeps decode steps out of graphs)
Block           expected_tensors(spec); __init__(spec, tensors, rt)
                graph_safe: bool   (every part of it is)
                forward(residual, pending, ctx, cache) -> (residual, pending)
                    ``pending`` is a delta not yet added to the residual, so that the next norm
                    can fuse the sum
Model           the top level, chosen by ``ModelSpec.kind``:
                expected_tensors(spec) -> every tensor the whole model reads (its own and its parts')
                __init__(spec, tensors, rt); graph_safe: bool
                cache_requirements() -> [CacheRequirement] one per schedule entry; bind_cache(manager)
                forward(ctx) -> float32 logits [n_wanted, vocab] at ctx.logit_rows, or None
                    ``DecoderModel`` ("decoder") is: token table -> blocks in schedule order -> final norm
                    on the wanted rows -> head; a top level that differs only at the two ends (a scaled
                    embedding, capped logits) derives from it and overrides ``embed`` / ``finish_logits``

No part knows which model it is in: sizes, constants and tensor names come from
its spec.  A new part registers itself with ``register_*`` (tests do so with toy
parts) and is then chosen by ``kind`` like the built-in ones.
"""

from __future__ import annotations

from ..weights.loader import ExpectedTensor

NORMS: dict[str, type] = {}
POSITIONS: dict[str, type] = {}
MIXERS: dict[str, type] = {}
FEEDFORWARDS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}
MODELS: dict[str, type] = {}


def _register(table: dict, what: str):
    def reg(kind: str, cls: type | None = None):
        def put(c):
            table[kind] = c
            return c
        return put(cls) if cls is not None else put
    reg.__doc__ = f"Register a {what} class under a spec ``kind`` (usable as a decorator)."
    return reg


register_norm = _register(NORMS, "norm")
register_position = _register(POSITIONS, "position encoding")
register_mixer = _register(MIXERS, "mixer")
register_feedforward = _register(FEEDFORWARDS, "feed-forward")
register_block = _register(BLOCKS, "block")
register_model = _register(MODELS, "model (top level)")


def _lookup(table: dict, kind: str, what: str) -> type:
    try:
        return table[kind]
    except KeyError:
        raise KeyError(f"no {what} registered for kind {kind!r}; known: {sorted(table)}") from None


def norm_class(spec): return _lookup(NORMS, spec.kind, "norm")
def position_class(spec): return _lookup(POSITIONS, spec.kind, "position encoding")
def mixer_class(spec): return _lookup(MIXERS, spec.kind, "mixer")
def feedforward_class(spec): return _lookup(FEEDFORWARDS, spec.kind, "feed-forward")
def block_class(spec): return _lookup(BLOCKS, spec.kind, "block")
def model_class(spec): return _lookup(MODELS, getattr(spec, "kind", "decoder"), "model")


def build_norm(spec, tensors, rt): return norm_class(spec)(spec, tensors, rt)
def build_position(spec, tensors, rt): return position_class(spec)(spec, tensors, rt)
def build_mixer(spec, tensors, rt): return mixer_class(spec)(spec, tensors, rt)
def build_feedforward(spec, tensors, rt): return feedforward_class(spec)(spec, tensors, rt)
def build_block(spec, tensors, rt): return block_class(spec)(spec, tensors, rt)
def build_model(spec, tensors, rt): return model_class(spec)(spec, tensors, rt)


def expected_tensors(model_spec) -> dict[str, ExpectedTensor]:
    """Every tensor the model reads, with its shape, in a fixed order; the top level named by
    ``model_spec.kind`` says which (its own and those of its parts)."""
    return model_class(model_spec).expected_tensors(model_spec)
