from . import attention, block, feedforward, model, norms, positions  # noqa: F401  (register the built-in parts)
from .attention import CacheView, PagedAttention
from .block import PreNormBlock
from .feedforward import GatedMLP
from .linear import Linear
from .model import DecoderModel
from .norms import RMSNorm
from .positions import NoPosition, Rotary, rotary_inv_freq, rotary_tables
from .registry import (
    BLOCKS,
    FEEDFORWARDS,
    MIXERS,
    MODELS,
    NORMS,
    POSITIONS,
    expected_tensors,
    register_block,
    register_feedforward,
    register_mixer,
    register_model,
    register_norm,
    register_position,
)
from .runtime import Runtime, Staging, Workspace
