"""Descriptions of a model as data: parts, blocks, and the order they run in.

A ``ModelSpec`` is what an architecture's ``config.json`` is turned into.  It
names every size and constant and every weight tensor, layer by layer, so that
two layers of one model may use different mixers, feed-forwards, norms or
position encodings.  Nothing here computes; the classes under ``parts`` are
built from these records through the registries in ``parts.registry``.

A new kind of part adds a frozen dataclass with a ``kind`` string here or in its
own module (tests define toy ones) and registers a class for that ``kind``.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of rotary embeddings, read from ``rope_scaling``."""

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis."""

    kind: str          # "rmsnorm"
    size: int
    eps: float
    weight: str        # tensor name of the gain


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer."""

    kind: str                     # "rotary" | "none"
    head_dim: int = 0
    theta: float = 0.0
    max_positions: int = 0
    scaling: RopeScaling | None = None


@dataclass(frozen=True)
class MixerSpec:
    """Base of token mixers; ``kind`` selects the registered class."""

    kind: str


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Causal grouped-query attention over a paged key/value cache."""

    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    window: int | None = None      # None: every earlier key; n: the last n keys, itself included
    position: PositionSpec = PositionSpec(kind="none")
    q_proj: str = ""
    k_proj: str = ""
    v_proj: str = ""
    o_proj: str = ""


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    """``down(act(gate(x)) * up(x))``."""

    hidden: int = 0
    intermediate: int = 0
    activation: str = "silu"
    gate_proj: str = ""
    up_proj: str = ""
    down_proj: str = ""


@dataclass(frozen=True)
class BlockSpec:
    """One residual block: which norm, mixer and feed-forward, and how arranged."""

    kind: str                      # "prenorm"
    mixer_norm: NormSpec
    mixer: MixerSpec
    ff_norm: NormSpec
    feedforward: FeedForwardSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.

    ``layer`` indexes ``ModelSpec.layers`` and may occur in several entries
    (shared weights).  ``cache_from`` names an EARLIER entry of the schedule whose
    cache this run reads instead of writing one of its own.
    """

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, layers, their order, final norm and head."""

    architecture: str
    vocab_size: int
    hidden: int
    max_positions: int
    embedding: str                           # tensor name of the token table
    layers: tuple[BlockSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    head: str | None                         # tensor name, or None: tied to the embedding
    optional_tensors: tuple[str, ...] = field(default_factory=tuple)  # present-but-unused names tolerated
    kind: str = "decoder"                    # which registered top level puts the parts together
