"""The engine: continuous batching over the step function, in the manner of the
reference's ``LlamaPagedEngine`` (engine/llama_paged_engine.py:106-455):
``submit`` / ``step`` / ``run_offline`` / ``has_work``, a page pool given as
``n_total_blocks`` x ``block_size``, an ``eos_token`` and a default sampling.

One ``step`` is one scheduler plan, one batch through the model (prompt
portions beside decode tokens), one sampling launch and one read of the
sampled ids.
"""

from __future__ import annotations

import gc
import tempfile
import time
from pathlib import Path

import torch

from .. import kernels
from ..config.registry import detect_config, get_preset
from ..sampling.sampler import Sampler, SamplingConfig, pack_rows, request_key
from ..weights.random_init import write_random_model
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import PLACEHOLDER, Request, Scheduler


class Engine:
    def __init__(self, runner: ModelRunner, eos_token=None, sampling: SamplingConfig | None = None,
                 max_queue_depth: int = 4096, max_batch: int | None = None, max_tokens_per_step: int = 2048,
                 chunk: int | None = None, pipeline: bool = True, trace_path: str | Path | None = None,
                 nvtx: bool = False):
        self.runner = runner
        self.cfg = sampling or SamplingConfig()
        if eos_token is None:
            eos_token = getattr(runner.config, "eos_token_id", None)
        self.eos = eos_token
        self.scheduler = Scheduler(runner.cache, runner.spec.max_positions,
                                   max_batch=max_batch or runner.cache.max_requests,
                                   max_tokens_per_step=max_tokens_per_step, chunk=chunk,
                                   max_queue_depth=max_queue_depth, eos_token=eos_token)
        self.sampler = Sampler(runner.rt)
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0}
        # One step ahead: a step is enqueued before the host has read the tokens of the step before; it
        # takes them on the device.  The host's work for a step then hides behind the GPU's work.
        self.pipeline = pipeline
        self._pending = None
        self._host_ids = [torch.empty(max(1, runner.cache.max_requests), dtype=torch.int32, pin_memory=True)
                          for _ in range(3)]
        self._host_next = 0
        # Observation, both off unless asked for: one JSON line per step (what the step was made of, pages free, the
        # host's time for it) into ``trace_path``, and an NVTX range around every step for a timeline tool.
        self._trace = open(trace_path, "w") if trace_path else None
        self._nvtx = bool(nvtx)

    def _observe(self, plan, t_host0: float, ahead: bool) -> None:
        if self._trace is None:
            return
        import json
        prefill = [e for e in plan.entries if not (len(e.tokens) == 1 and e.request.generated)]
        rec = {"step": self.stats["steps"], "requests": len(plan.entries), "tokens": sum(len(e.tokens) for e in plan.entries),
               "prefill_tokens": sum(len(e.tokens) for e in prefill), "decode_tokens": len(plan.entries) - len(prefill),
               "sampled": sum(1 for e in plan.entries if e.wants_logits), "preempted": len(plan.preempted),
               "running": len(self.scheduler.running), "queued": len(self.scheduler.queue),
               "pages_free": self.runner.cache.n_free_pages(), "graph_replays": self.runner.graphs.replays,
               "enqueued_ahead": ahead, "host_us": round((time.perf_counter() - t_host0) * 1e6, 1)}
        self._trace.write(json.dumps(rec) + "\n")
        self._trace.flush()

    # ------------------------------------------------------------ construction
    @classmethod
    def from_dir(cls, model_dir: str | Path, dtype="bfloat16", device="cuda:0", n_total_blocks: int = 4096,
                 block_size: int = 16, max_requests: int = 64, **kw) -> "Engine":
        runner = ModelRunner.from_dir(model_dir, dtype=dtype, device=device, page_size=block_size,
                                      n_pages=n_total_blocks, max_requests=max_requests)
        return cls(runner, **kw)

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype="bfloat16", store_dtype: str = "bfloat16", **kw) -> "Engine":
        """An engine over random weights: the model folder is written to a temporary
        place with the random-weights mode and loaded like any other."""
        if isinstance(config, str):
            config = get_preset(config)
        with tempfile.TemporaryDirectory(prefix="inf_engine_random_") as tmp:
            write_random_model(config, seed, tmp, store_dtype=store_dtype)
            return cls.from_dir(tmp, dtype=dtype, **kw)

    # ------------------------------------------------------------------ queue
    def submit(self, req: Request) -> bool:
        if not req.arrival_time:
            req.arrival_time = time.perf_counter()      # the clock that run_offline and generate step with
        return self.scheduler.submit(req)

    @staticmethod
    def latency_stats(requests: list[Request]) -> dict:
        """Time to the first token and time per later token over finished requests: mean, median and worst, in
        seconds, and the per-request figures."""
        def summary(values):
            v = sorted(x for x in values if x is not None)
            if not v:
                return None
            return {"mean": sum(v) / len(v), "p50": v[len(v) // 2], "max": v[-1]}
        per = [{"req_id": r.req_id, "prompt_tokens": len(r.prompt_ids), "new_tokens": len(r.generated),
                "ttft_s": r.ttft, "tpot_s": r.tpot, "preemptions": r.preemptions} for r in requests if r.finish_time]
        return {"ttft_s": summary(p["ttft_s"] for p in per), "tpot_s": summary(p["tpot_s"] for p in per), "requests": per}

    @property
    def has_work(self) -> bool:
        return self.scheduler.has_work or self._pending is not None

    @property
    def completed(self) -> list[Request]:
        return self.scheduler.completed

    # ------------------------------------------------------------------- step
    @torch.no_grad()
    def step(self, now: float = 0.0) -> list[Request]:
        """Admit, run one mixed batch, sample, finish; returns the requests completed.

        With ``pipeline`` the step is enqueued before the tokens of the step before are read (they are
        taken on the device), and the requests returned are those that the step BEFORE completed."""
        if self._nvtx:
            torch.cuda.nvtx.range_push(f"engine step {self.stats['steps']}")
        try:
            if self.pipeline and self._can_pipeline():
                return self._step_ahead(now)
            done = self._drain(now)
            return done + self._step_now(now)
        finally:
            if self._nvtx:
                torch.cuda.nvtx.range_pop()

    # a penalty over generated tokens needs them on the host; so does a plan that may have to preempt
    def _can_pipeline(self) -> bool:
        s = self.scheduler
        if self.cfg.repetition_penalty != 1.0:
            return False
        for r in list(s.running) + s.queue[:4]:
            if r.sampling is not None and r.sampling.repetition_penalty != 1.0:
                return False
        return s.cache.n_free_pages() >= len(s.running) + 1

    def _drain(self, now: float) -> list[Request]:
        if self._pending is None:
            return []
        pend, self._pending = self._pending, None
        return self._resolve(pend, None, now)

    def _resolve(self, pend, in_flight, now: float) -> list[Request]:
        plan, wanted, host, event = pend["plan"], pend["wanted"], pend["host"], pend["event"]
        event.synchronize()                                   # the step's one device-to-host read has landed
        ids = host[:len(wanted)].tolist()
        return self.scheduler.resolve(plan, {e.request.req_id: t for e, t in zip(wanted, ids)}, in_flight, now)

    def _step_ahead(self, now: float) -> list[Request]:
        t_host0 = time.perf_counter()
        prev = self._pending
        plan = self.scheduler.plan()
        self.stats["preemptions"] += len(plan.preempted)
        if not plan.entries:
            return self._drain(now)
        prev_index = {e.request.req_id: i for i, e in enumerate(prev["wanted"])} if prev else {}
        entries, token_src, any_src = [], [], False
        for e in plan.entries:
            toks = e.tokens
            if toks[-1] == PLACEHOLDER:                       # the token the step before sampled for this request
                assert len(toks) == 1 and e.request.req_id in prev_index
                token_src.append(prev_index[e.request.req_id])
                toks = [0]
                any_src = True
            else:
                token_src.extend([-1] * len(toks))
            entries.append(StepEntry(e.request.req_id, toks, [len(toks) - 1] if e.wants_logits else []))
        wanted = [e for e in plan.entries if e.wants_logits]
        configs = [e.request.sampling or self.cfg for e in wanted]
        keys = [request_key(e.request.req_id, len(e.request.generated)) for e in wanted]
        rows = pack_rows(configs, keys, self.runner.spec.vocab_size) if wanted else None
        _, ids = self.runner.step_and_sample(entries, rows, device_tokens=prev["dev"] if any_src else None,
                                             token_src=token_src if any_src else None)
        for e in plan.entries:
            self.stats["decode_tokens" if len(e.tokens) == 1 and e.request.generated else "prefill_tokens"] += len(e.tokens)
        self.stats["steps"] += 1
        self._observe(plan, t_host0, True)
        self.scheduler.book(plan)
        new = None
        if wanted:
            host = self._host_ids[self._host_next]
            self._host_next = (self._host_next + 1) % len(self._host_ids)
            host[:len(wanted)].copy_(ids[:len(wanted)], non_blocking=True)
            event = torch.cuda.Event()
            event.record()
            new = {"plan": plan, "wanted": wanted, "host": host, "event": event, "dev": ids}
        done = self._resolve(prev, plan, now) if prev else []      # read the step before while this one runs
        self._pending = new
        return done

    def _step_now(self, now: float) -> list[Request]:
        t_host0 = time.perf_counter()
        plan = self.scheduler.plan()
        self.stats["preemptions"] += len(plan.preempted)
        if not plan.entries:
            return []
        entries = [StepEntry(e.request.req_id, e.tokens, [len(e.tokens) - 1] if e.wants_logits else [])
                   for e in plan.entries]
        sampled = {}
        wanted = [e for e in plan.entries if e.wants_logits]
        configs = [e.request.sampling or self.cfg for e in wanted]
        keys = [request_key(e.request.req_id, len(e.request.generated)) for e in wanted]
        if wanted and all(c.repetition_penalty == 1.0 for c in configs):
            # sampling rides in the step (inside the CUDA graph of a decode step)
            rows = pack_rows(configs, keys, self.runner.spec.vocab_size)
            _, ids = self.runner.step_and_sample(entries, rows)
        else:
            logits = self.runner.step(entries)
            ids = None
            if wanted:
                contexts = [e.request.generated for e in wanted]
                ids = self.sampler.sample(logits, configs, keys, contexts)
        if wanted:
            ids = ids.tolist()                                   # the step's one device-to-host read
            sampled = {e.request.req_id: t for e, t in zip(wanted, ids)}
        for e in plan.entries:
            self.stats["decode_tokens" if len(e.tokens) == 1 and e.request.generated else "prefill_tokens"] += len(e.tokens)
        self.stats["steps"] += 1
        self._observe(plan, t_host0, False)
        return self.scheduler.commit(plan, sampled, now)

    def run_offline(self, requests: list[Request]) -> dict[int, list[int]]:
        """Submit everything, run to completion; ``{req_id: generated}``
        (engine/llama_paged_engine.py:445-455).  Requests refused at submit map to []."""
        refused = [r for r in requests if not self.submit(r)]
        # A decode step is some 50 us of host work in front of a millisecond of GPU work; a full collection of the
        # host's garbage (10 ms and more with a model's objects to walk) in the middle of the run leaves the GPU
        # without launches for ten steps.  What exists now is set aside from the collector for the run.
        gc.collect()
        gc.freeze()
        try:
            while self.has_work:
                self.step(time.perf_counter())
        finally:
            gc.unfreeze()
        kernels.check_device_errors()
        out = {r.req_id: r.generated for r in self.completed}
        out.update({r.req_id: [] for r in refused})
        return out

    def generate(self, prompt_ids: list[int], max_new_tokens: int, sampling: SamplingConfig | None = None,
                 req_id: int = 0) -> list[int]:
        """Continuation of one prompt (the reference's ``generate_cached``, engine/llama_model.py:177-215)."""
        if max_new_tokens <= 0:
            return []
        req = Request(req_id=req_id, prompt_ids=list(prompt_ids), max_new_tokens=max_new_tokens, sampling=sampling)
        if not self.submit(req):
            raise ValueError(f"request refused: {req.error}")
        while req not in self.completed:
            self.step(time.perf_counter())
        self.completed.remove(req)
        kernels.check_device_errors()
        return req.generated


def load_engine(model_dir_or_preset: str, dtype="bfloat16", random_weights: bool = False, seed: int = 0, **kw) -> Engine:
    """An engine from a model folder, or from a preset name with random weights."""
    p = Path(model_dir_or_preset)
    if p.is_dir() and not random_weights:
        return Engine.from_dir(p, dtype=dtype, **kw)
    return Engine.from_random(get_preset(model_dir_or_preset), seed=seed, dtype=dtype, **kw)


__all__ = ["Engine", "Request", "load_engine", "detect_config"]
