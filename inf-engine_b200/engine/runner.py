"""The step function: a model, its cache, and ``step(entries) -> logits``.

``ModelRunner`` is what generation, the scheduler and trace replay all drive.
A step reserves pages for the tokens it brings, runs only those tokens as one
batch against the cache that earlier steps left, advances the requests'
lengths, and returns float32 logits at the wanted places, in the order of the
entries and of their ``want`` lists.
"""

from __future__ import annotations

from pathlib import Path

import torch

from .. import kernels
from ..cache.manager import CacheManager
from ..config.registry import detect_config
from ..parts.registry import build_model, expected_tensors
from ..parts.runtime import Runtime
from ..weights.loader import load_weights
from .batch import StepEntry, build_context
from .graphs import DecodeGraphs

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class OutOfPages(RuntimeError):
    """The step's tokens do not fit the free pages; nothing was run or taken."""


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}") from None


class ModelRunner:
    def __init__(self, config, tensors: dict, dtype, device="cuda:0", page_size: int = 16, n_pages: int = 256,
                 max_requests: int = 64, spec=None, use_graphs: bool = True, poison_free_pages: bool = False):
        self.config = config
        self.spec = spec if spec is not None else config.model_spec()
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.rt = Runtime(self.device, self.dtype)
        self.model = build_model(self.spec, tensors, self.rt)     # the top level that spec.kind names
        max_pages_per_request = -(-self.spec.max_positions // page_size)
        self.cache = CacheManager(self.model.cache_requirements(), page_size, n_pages, max_requests,
                                  min(n_pages, max_pages_per_request))
        self.cache.poison_free_pages = poison_free_pages      # a debugging aid: NaN in every page that nobody holds
        self.cache.allocate_storage(self.device)
        self.model.bind_cache(self.cache)
        if kernels.checks_enabled():
            # a checks build compares every page id, slot and token id the kernels read with this pool and vocabulary
            kernels.set_check_limits(n_pages, n_pages * page_size, self.spec.vocab_size)
        self.page_size = page_size
        self.steps = 0
        self.use_graphs = use_graphs
        self.graphs = DecodeGraphs(self)

    # ------------------------------------------------------------ construction
    @classmethod
    def from_dir(cls, model_dir: str | Path, dtype="bfloat16", device="cuda:0", **kw) -> "ModelRunner":
        config = detect_config(model_dir)
        spec = config.model_spec()
        run_dtype = parse_dtype(dtype)
        tensors = load_weights(model_dir, expected_tensors(spec), run_dtype, device, optional=spec.optional_tensors)
        return cls(config, tensors, run_dtype, device, spec=spec, **kw)

    # ------------------------------------------------------------------ steps
    def open(self, rid) -> bool:
        """Make ``rid`` known to the cache; False when every request slot is in use."""
        return self.cache.open(rid) is not None

    def close(self, rid) -> None:
        self.cache.close(rid)

    def is_open(self, rid) -> bool:
        return rid in self.cache.slots

    def length(self, rid) -> int:
        return self.cache.lengths[rid]

    def step(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """Run one batch.  Returns float32 logits [n_wanted, vocab] on the device
        (a view of a buffer that the next step overwrites) or None."""
        return self.step_and_sample(entries, None)[0]

    def step_and_sample(self, entries: list[StepEntry], sample_rows=None, device_tokens=None, token_src=None):
        """``step`` plus, when ``sample_rows`` (int32 numpy [n_wanted, 7] records of
        ``sampling.Sampler.pack``) is given, the sampled token ids (int32, device).
        Steps that are all single decode tokens replay a CUDA graph.  ``device_tokens`` (int32 on the
        device) with ``token_src`` (per token of the step an index into it, or -1) replaces token ids that
        the host does not know yet; without ``token_src`` it replaces all of them in order."""
        if not entries:
            return None, None
        cache = self.cache
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if e.rid not in cache.slots:
                raise KeyError(f"request {e.rid!r} is not open")
            new_len = cache.lengths[e.rid] + len(e.tokens)
            if new_len > self.spec.max_positions:
                raise ValueError(f"request {e.rid!r} would reach {new_len} tokens, beyond max_positions="
                                 f"{self.spec.max_positions}")
            for t in e.tokens:
                if not 0 <= t < self.spec.vocab_size:
                    raise ValueError(f"token id {t} of request {e.rid!r} is outside the vocabulary")
        # all or nothing: check first, then take
        need = [0] * len(cache.kv_groups)
        for e in entries:
            for gi, n in enumerate(cache.pages_needed(e.rid, cache.lengths[e.rid] + len(e.tokens))):
                need[gi] += n
        for gi, g in enumerate(cache.kv_groups):
            if need[gi] > g.pool.n_free:
                raise OutOfPages(f"step needs {need[gi]} pages of group {gi}, {g.pool.n_free} are free")
        for e in entries:
            ok = cache.reserve(e.rid, cache.lengths[e.rid] + len(e.tokens))
            assert ok
        sampled = None
        if self.use_graphs and self.graphs.usable(entries):
            logits, sampled = self.graphs.step(entries, sample_rows, device_tokens, token_src)
        else:
            ctx = build_context(self.rt, cache, entries)
            if device_tokens is not None:
                if token_src is None:
                    ctx.token_ids.copy_(device_tokens)
                else:
                    import numpy as np
                    from .. import kernels
                    src = self.rt.staging.upload(np.asarray(token_src, dtype=np.int32))
                    kernels.patch_tokens(ctx.token_ids, src, device_tokens)
            logits = self.model.forward(ctx)
            if sample_rows is not None and logits is not None:
                from .. import kernels
                rows = self.rt.staging.upload(sample_rows.reshape(-1)).view(-1, 7)
                sampled = self.rt.ws.take("sampled", (logits.shape[0],), torch.int32)
                kernels.sample(logits, rows, sampled)
        for e in entries:
            cache.advance(e.rid, cache.lengths[e.rid] + len(e.tokens))
        self.steps += 1
        return logits, sampled
