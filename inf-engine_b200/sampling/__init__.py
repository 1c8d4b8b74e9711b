from .sampler import (
    REPETITION_PENALTY_WINDOW,
    Sampler,
    SamplingConfig,
    SamplingMode,
    request_key,
    splitmix64,
    uniform_of,
)
