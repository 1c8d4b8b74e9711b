"""B200-native inference engine for the dense Llama decoder (Llama 3.2, SmolLM2).

Public surface, in the manner of the reference's ``engine`` package
(engine/__init__.py:39-112):

    from inf_engine_b200 import Engine, Request, SamplingConfig, SamplingMode
    engine = Engine.from_dir(model_dir, dtype="bfloat16", n_total_blocks=4096, block_size=16)
    out = engine.run_offline([Request(req_id=0, prompt_ids=[1, 2, 3], max_new_tokens=16)])

The reference's names ``LlamaPagedEngine`` and ``LlamaRequest`` are kept as aliases.
"""

from .cache import CacheManager, CacheRequirement, PagePool
from .config import (
    ConfigError,
    LlamaConfig,
    ModelSpec,
    detect_config,
    get_llama_config,
    get_preset,
    parse_config_dict,
    register_architecture,
)
from .engine import Engine, ModelRunner, OutOfPages, Request, Scheduler, StepEntry, load_engine
from .sampling import SamplingConfig, SamplingMode
from .weights import WeightsError, load_weights, write_random_model

LlamaPagedEngine = Engine
LlamaRequest = Request

__all__ = [
    "CacheManager", "CacheRequirement", "ConfigError", "Engine", "LlamaConfig", "LlamaPagedEngine",
    "LlamaRequest", "ModelRunner", "ModelSpec", "OutOfPages", "PagePool", "Request", "SamplingConfig",
    "SamplingMode", "Scheduler", "StepEntry", "WeightsError", "detect_config", "get_llama_config", "get_preset",
    "load_engine", "load_weights", "parse_config_dict", "register_architecture", "write_random_model",
]
