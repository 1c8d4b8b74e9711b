"""Typed configuration of the dense Llama decoder, read from ``config.json``.

The reference keeps these numbers in a frozen dataclass with presets
(engine/config.py:13-133) and only a diagnostic script maps ``config.json`` keys
to its fields (scripts/inspect_model.py:92-108).  Here the file's own keys are
the fields; the reference's short names are offered as read-only aliases.
"""

from __future__ import annotations

from dataclasses import dataclass, asdict

from .spec import (
    AttentionSpec,
    BlockSpec,
    GatedMLPSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    RopeScaling,
    ScheduleEntry,
)


class ConfigError(ValueError):
    """A ``config.json`` that is incomplete, inconsistent, or asks for what is not built."""


_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "num_hidden_layers",
    "num_attention_heads",
    "intermediate_size",
    "max_position_embeddings",
)


@dataclass(frozen=True)
class LlamaConfig:
    """Every size and constant of a ``LlamaForCausalLM`` checkpoint.

    Defaults of the optional keys: ``rms_norm_eps`` 1e-5 and an untied head as in
    the reference's dataclass (engine/config.py:42-44).  A ``config.json`` without
    ``rope_theta`` means 10000, the value that checkpoints of this architecture had
    before the key existed (the reference's 500000 is the default of its presets,
    which name it).  ``head_dim`` defaults to ``hidden_size // num_attention_heads``
    (engine/config.py:60-66).
    """

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    max_position_embeddings: int
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling | None = None
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    eos_token_id: int | tuple[int, ...] | None = None
    bos_token_id: int | None = None
    torch_dtype: str | None = None

    # ---- the reference's names (engine/config.py:27-44) as aliases
    @property
    def d_model(self) -> int:
        return self.hidden_size

    @property
    def n_layer(self) -> int:
        return self.num_hidden_layers

    @property
    def n_head(self) -> int:
        return self.num_attention_heads

    @property
    def n_kv_heads(self) -> int:
        return self.num_key_value_heads

    @property
    def n_kv_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def n_ctx(self) -> int:
        return self.max_position_embeddings

    @property
    def norm_eps(self) -> float:
        return self.rms_norm_eps

    # ---- reading and writing config.json
    @classmethod
    def from_hf_dict(cls, d: dict) -> "LlamaConfig":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {', '.join(missing)}")
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        n_head = int(d["num_attention_heads"])
        hidden = int(d["hidden_size"])
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % n_head:
                raise ConfigError(f"hidden_size={hidden} is not divisible by num_attention_heads={n_head}")
            head_dim = hidden // n_head
        scaling = d.get("rope_scaling")
        rope_scaling = None
        if scaling:
            kind = scaling.get("rope_type", scaling.get("type"))
            if kind in (None, "default"):
                rope_scaling = None
            elif kind == "llama3":
                try:
                    rope_scaling = RopeScaling(
                        rope_type="llama3",
                        factor=float(scaling["factor"]),
                        low_freq_factor=float(scaling["low_freq_factor"]),
                        high_freq_factor=float(scaling["high_freq_factor"]),
                        original_max_position_embeddings=int(scaling["original_max_position_embeddings"]),
                    )
                except KeyError as e:
                    raise ConfigError(f"rope_scaling of type llama3 lacks key {e}") from None
            else:
                raise ConfigError(f"rope_scaling type {kind!r} is not built (known: llama3, default)")
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = tuple(int(e) for e in eos)
        cfg = cls(
            architecture=str(archs[0]),
            vocab_size=int(d["vocab_size"]),
            hidden_size=hidden,
            num_hidden_layers=int(d["num_hidden_layers"]),
            num_attention_heads=n_head,
            num_key_value_heads=int(d.get("num_key_value_heads") or n_head),
            head_dim=int(head_dim),
            intermediate_size=int(d["intermediate_size"]),
            max_position_embeddings=int(d["max_position_embeddings"]),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=rope_scaling,
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
            eos_token_id=eos,
            bos_token_id=d.get("bos_token_id"),
            torch_dtype=d.get("torch_dtype", d.get("dtype")),
        )
        if d.get("attention_bias") or d.get("mlp_bias"):
            raise ConfigError("attention_bias / mlp_bias are not built: the reference's Llama has no biases")
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "intermediate_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            # engine/config.py:71-72
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not divisible by "
                f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotary embeddings")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act={self.hidden_act!r} is not built (the reference fixes SiLU)")
        if self.rms_norm_eps <= 0:
            raise ConfigError("rms_norm_eps must be positive")
        if self.rope_scaling is not None:
            s = self.rope_scaling
            if s.factor <= 0 or s.high_freq_factor <= s.low_freq_factor or s.original_max_position_embeddings <= 0:
                raise ConfigError(f"inconsistent rope_scaling: {s}")

    def to_hf_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        if isinstance(d["eos_token_id"], tuple):
            d["eos_token_id"] = list(d["eos_token_id"])
        d = {k: v for k, v in d.items() if v is not None or k == "rope_scaling"}
        return d

    # ---- the model as data
    def model_spec(self) -> ModelSpec:
        """The Llama decoder: L identical pre-norm blocks, each run once, in order
        (engine/llama_model.py:139-149, engine/llama_block.py:50-62)."""
        position = PositionSpec(
            kind="rotary",
            head_dim=self.head_dim,
            theta=self.rope_theta,
            max_positions=self.max_position_embeddings,
            scaling=self.rope_scaling,
        )
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            layers.append(
                BlockSpec(
                    kind="prenorm",
                    mixer_norm=NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps, p + "input_layernorm.weight"),
                    mixer=AttentionSpec(
                        kind="attention",
                        hidden=self.hidden_size,
                        n_heads=self.num_attention_heads,
                        n_kv_heads=self.num_key_value_heads,
                        head_dim=self.head_dim,
                        window=None,
                        position=position,
                        q_proj=p + "self_attn.q_proj.weight",
                        k_proj=p + "self_attn.k_proj.weight",
                        v_proj=p + "self_attn.v_proj.weight",
                        o_proj=p + "self_attn.o_proj.weight",
                    ),
                    ff_norm=NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps,
                                     p + "post_attention_layernorm.weight"),
                    feedforward=GatedMLPSpec(
                        kind="gated_mlp",
                        hidden=self.hidden_size,
                        intermediate=self.intermediate_size,
                        activation=self.hidden_act,
                        gate_proj=p + "mlp.gate_proj.weight",
                        up_proj=p + "mlp.up_proj.weight",
                        down_proj=p + "mlp.down_proj.weight",
                    ),
                )
            )
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding="model.embed_tokens.weight",
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(layer=i) for i in range(self.num_hidden_layers)),
            final_norm=NormSpec("rmsnorm", self.hidden_size, self.rms_norm_eps, "model.norm.weight"),
            head=None if self.tie_word_embeddings else "lm_head.weight",
            # a tied checkpoint may still carry lm_head.weight; the tie wins (engine/llama_weights.py:45-47)
            optional_tensors=("lm_head.weight",) if self.tie_word_embeddings else (),
        )
