from .llama import ConfigError, LlamaConfig
from .registry import (
    ARCHITECTURES,
    Architecture,
    detect_config,
    get_architecture,
    get_llama_config,
    get_preset,
    parse_config_dict,
    preset_names,
    register_architecture,
)
from .spec import (
    AttentionSpec,
    BlockSpec,
    FeedForwardSpec,
    GatedMLPSpec,
    MixerSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    RopeScaling,
    ScheduleEntry,
)
