from .sampler import (
    REPETITION_PENALTY_WINDOW,
    Sampler,
    SamplingConfig,
    SamplingMode,
    pack_rows,
    request_key,
    splitmix64,
    uniform_of,
)
