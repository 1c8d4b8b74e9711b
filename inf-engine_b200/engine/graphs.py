"""Decode steps as CUDA graphs.

A decode step (one token for each of R requests) is a few hundred short
launches; replaying them as one graph removes the launch gaps that otherwise
dominate at small batch.  The reference does the same with
``torch.cuda.CUDAGraph`` per (batch, length) bucket and ``.copy_()`` into static
tensors (engine/llama_paged_engine.py:288-415).

Here a graph is kept per (batch bucket, block-table width).  Everything that
changes from step to step — token ids, positions, lengths, page slots, block
tables, sampling records — sits in one static int32 buffer that is refilled by
a single copy from pinned memory before each replay; kernels read lengths and
tables from it, so one graph serves every context length.  Rows beyond the
live requests are padding: length 0, no page, their results are ignored.
The graph also holds the sampling kernel, so a step returns token ids.
"""

from __future__ import annotations

import gc

import numpy as np
import torch

from ..parts.runtime import Workspace
from .batch import KVGroupContext, StepContext

BATCH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def _bucket(n: int, choices) -> int | None:
    for c in choices:
        if c >= n:
            return c
    return None


def keys_bucket(keys: int) -> int:
    """The longest context a graph is cut for, given the step's: the next multiple of KEYS_STEP up to 4,096 keys, of a
    sixteenth of the power of two below beyond that.  The decode attention's split is part of the captured launch, so a
    graph cut for more keys than the step has leaves some of its warps without keys (at most a sixteenth of them
    here), and every new bucket is a capture of some 20 ms: a capture per 256 keys of a context of 32,768 would be
    one every 256 steps for good."""
    step = KEYS_STEP
    if keys > 16 * KEYS_STEP:
        step = (1 << (int(keys - 1).bit_length() - 1)) // 16
    return -(-keys // step) * step


class _Captured:
    def __init__(self):
        self.graph = None
        self.generation = -1


KEYS_STEP = 256      # graphs are captured per this many keys of the longest context (more when it is long: keys_bucket)
MAX_GRAPHS = 48      # captured graphs kept; the one unused for longest goes first


class DecodeGraphs:
    def __init__(self, runner):
        self.runner = runner
        self.rt = runner.rt
        self.ws = Workspace(self.rt.device)          # buffers that captured graphs point into
        self.generation = 0
        self._buckets: dict = {}
        self.replays = 0
        self.captures = 0
        self._capture_stream = None

    def usable(self, entries) -> bool:
        if not self.runner.model.graph_safe:
            return False
        if len(entries) > BATCH_BUCKETS[-1]:
            return False
        return all(len(e.tokens) == 1 and e.want == [0] for e in entries)

    # ---------------------------------------------------------------- layout
    def _layout(self, B: int, widths: tuple[int, ...]):
        off = {}
        n = 0
        for name in ("token_ids", "positions", "ctx_before", "slots"):
            off[name] = (n, B)
            n += B
        for g, w in enumerate(widths):
            off[f"slot_mapping{g}"] = (n, B)
            n += B
            off[f"block_table{g}"] = (n, B * w)
            n += B * w
        off["sample_rows"] = (n, B * 7)
        n += B * 7
        off["token_src"] = (n, B)
        n += B
        return off, n

    def _get(self, B: int, widths: tuple[int, ...], keys_hint: int):
        key = (B, widths, keys_hint)
        b = self._buckets.get(key)
        if b is not None:
            self._buckets[key] = self._buckets.pop(key)       # most recently used last
        if b is None:
            while len(self._buckets) >= MAX_GRAPHS:
                self._buckets.pop(next(iter(self._buckets)))
            b = _Captured()
            b.B, b.widths = B, widths
            b.off, b.n = self._layout(B, widths)
            b.dev = torch.zeros(b.n, dtype=torch.int32, device=self.rt.device)
            b.host = np.zeros(b.n, dtype=np.int32)
            dev = self.rt.device
            ctx = StepContext(self.rt, self.runner.page_size)
            view = lambda name: b.dev[b.off[name][0]:b.off[name][0] + b.off[name][1]]
            ctx.token_ids, ctx.positions = view("token_ids"), view("positions")
            ctx.ctx_before, ctx.slots = view("ctx_before"), view("slots")
            ctx.q_start = torch.arange(B + 1, dtype=torch.int32, device=dev)
            ctx.logit_rows = torch.arange(B, dtype=torch.int32, device=dev)
            ctx.kv = [KVGroupContext(view(f"slot_mapping{g}"), view(f"block_table{g}").view(B, w))
                      for g, w in enumerate(widths)]
            ctx.n_tokens = ctx.n_requests = ctx.n_logits = B
            ctx.max_q_len = 1
            ctx.keys_cap = min(keys_hint, min(widths) * self.runner.page_size) if widths else 0
            ctx.host = {"q_lens": [1] * B, "q_start": list(range(B + 1)), "slots": [0] * B, "graph": True}
            b.ctx = ctx
            b.rows = view("sample_rows").view(B, 7)
            b.token_src = view("token_src")
            b.sampled = torch.zeros(B, dtype=torch.int32, device=dev)
            b.logits = None
            self._buckets[key] = b
        return b

    # ------------------------------------------------------------------ steps
    def _fill(self, b, entries, sample_rows: np.ndarray | None, token_src=None) -> None:
        cache = self.runner.cache
        ps = cache.page_size
        B, R = b.B, len(entries)
        h = b.host
        h[:] = 0
        o = b.off
        lens = np.fromiter((cache.lengths[e.rid] for e in entries), dtype=np.int32, count=R)
        h[o["token_ids"][0]:o["token_ids"][0] + R] = [e.tokens[0] for e in entries]
        h[o["positions"][0]:o["positions"][0] + R] = lens
        h[o["ctx_before"][0]:o["ctx_before"][0] + R] = lens
        h[o["slots"][0]:o["slots"][0] + R] = [cache.slots[e.rid] for e in entries]
        for g, w in enumerate(b.widths):
            grp = cache.kv_groups[g]
            s0 = o[f"slot_mapping{g}"][0]
            t0 = o[f"block_table{g}"][0]
            h[s0:s0 + B] = -1
            table = h[t0:t0 + B * w].reshape(B, w)
            table[:] = -1
            for r, e in enumerate(entries):
                t = grp.tables[e.rid]
                table[r, :len(t)] = t
                p = int(lens[r])
                h[s0 + r] = t[p // ps] * ps + p % ps
        if sample_rows is not None:
            r0 = o["sample_rows"][0]
            rows = h[r0:r0 + B * 7].reshape(B, 7)
            rows[:R] = sample_rows
            rows.view(np.float32)[R:, 1] = 1.0      # padding rows: greedy
        t0 = o["token_src"][0]
        h[t0:t0 + B] = -1
        if token_src is not None:
            h[t0:t0 + R] = token_src
        self.rt.staging.upload(h, into=b.dev)

    def _forward(self, b):
        from .. import kernels
        logits = self.runner.model.forward(b.ctx)
        kernels.sample(logits, b.rows, b.sampled)
        return logits

    def step(self, entries, sample_rows: np.ndarray | None, device_tokens: torch.Tensor | None = None,
             token_src=None):
        """Run one decode step for ``entries`` (pages reserved by the caller).
        Returns (logits [R, V], sampled ids [R] or None), views of static buffers.
        ``device_tokens`` (int32 [R] on the device, e.g. the ids the last step sampled)
        replaces the entries' token ids without a trip through the host: all of them, or, with
        ``token_src`` (one index into ``device_tokens`` per entry, -1 to keep the host's id), some."""
        cache = self.runner.cache
        R = len(entries)
        B = _bucket(R, BATCH_BUCKETS)
        widths = tuple(_bucket(max(len(g.tables[e.rid]) for e in entries), [1 << i for i in range(3, 24)])
                       for g in cache.kv_groups)
        # the split-key attention is cut for the longest context of the step, in steps of KEYS_STEP keys: a
        # graph serves until some request has grown past its step
        keys_hint = keys_bucket(max(cache.lengths[e.rid] for e in entries) + 1)
        b = self._get(B, widths, keys_hint)
        self._fill(b, entries, sample_rows, token_src)
        if device_tokens is not None:
            if token_src is None:
                b.ctx.token_ids[:R].copy_(device_tokens[:R])
            else:
                from .. import kernels
                kernels.patch_tokens(b.ctx.token_ids[:R], b.token_src, device_tokens)
        rt = self.rt
        saved = rt.ws
        rt.ws = self.ws
        try:
            if b.graph is None or b.generation != self.generation:
                # warm-up outside capture (sizes the buffers, builds the work lists), then capture
                before = self.ws.moves
                cs = self._capture_stream
                if cs is None:
                    cs = self._capture_stream = torch.cuda.Stream()
                cs.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(cs):
                    self._forward(b)
                torch.cuda.current_stream().wait_stream(cs)
                torch.cuda.synchronize()
                if self.ws.moves != before:
                    # a buffer was replaced by a larger one: graphs captured earlier point at freed memory.  (A buffer
                    # that is new leaves them alone: the first step of at most 16 requests brings buffers of its own,
                    # and throwing the graphs of the larger steps away for that cost a run of 32 requests 0.1 s.)
                    self.generation += 1
                from .. import kernels
                g = torch.cuda.CUDAGraph()
                n0 = kernels.LAUNCHES
                # The collector must not run inside the capture: garbage that owns CUDA objects (an engine
                # dropped earlier, with graphs of its own) would free them there, which a capture forbids and
                # which invalidates it.  So the collector is held until the capture ends.  The capture is begun
                # and ended by hand: torch.cuda.graph() would first run a full collection and empty the
                # allocator's cache, tens of milliseconds for every graph of a long generation.
                gc_was_on = gc.isenabled()
                gc.disable()
                try:
                    with torch.cuda.stream(cs):
                        g.capture_begin(capture_error_mode="thread_local")
                        try:
                            b.logits = self._forward(b)
                        finally:
                            g.capture_end()
                finally:
                    if gc_was_on:
                        gc.enable()
                torch.cuda.current_stream().wait_stream(cs)
                b.n_kernels = kernels.LAUNCHES - n0
                b.graph, b.generation = g, self.generation
                self.captures += 1
            from .. import kernels
            b.graph.replay()                      # capture recorded the launches; this runs them
            kernels.LAUNCHES += b.n_kernels
            self.replays += 1
        finally:
            rt.ws = saved
        return b.logits[:R], (b.sampled[:R] if sample_rows is not None else None)
