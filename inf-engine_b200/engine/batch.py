"""The batch of one step: for each request a run of its next tokens, flattened.

The reference's forward takes a rectangle (B, T) and its engine feeds it either
one whole prompt or one token per active request
(engine/llama_paged_engine.py:199-202, 242-257).  Here a step is a flat list of
tokens cut anywhere: a request contributes ``q_len >= 1`` consecutive tokens
that start at its current length.  Everything the kernels need to know about
the batch is a handful of int32 arrays that go to the device in one copy.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepEntry:
    """One request's share of a step."""

    rid: object
    tokens: list[int]
    want: list[int] = field(default_factory=list)   # indices into ``tokens`` whose logits are asked for


@dataclass
class KVGroupContext:
    slot_mapping: torch.Tensor      # int32 [N]: page*page_size + offset of every token of the step
    block_table: torch.Tensor       # int32 [R, width]: page ids of every request, -1 where none


class StepContext:
    """Device-side description of a step plus the host copy parts may consult.

    Device tensors (int32): ``token_ids[N]``, ``positions[N]``, ``q_start[R+1]``,
    ``ctx_before[R]`` (tokens a request held before the step), ``slots[R]``
    (per-request state slot), ``logit_rows[M]``; per kv group ``slot_mapping[N]``
    and ``block_table[R, width]``.  Host lists of the same names live in
    ``host``.
    """

    def __init__(self, rt, page_size: int):
        self.rt = rt
        self.page_size = page_size
        self.n_tokens = 0
        self.n_requests = 0
        self.n_logits = 0
        self.host: dict = {}
        self.kv: list[KVGroupContext] = []
        self.token_ids = self.positions = self.q_start = self.ctx_before = self.slots = self.logit_rows = None
        self._work: dict = {}
        self.max_q_len = 0
        self.max_seq_len = 0
        self.keys_cap = 0          # no request of the step holds more keys than this (sizes split-key grids)
        # scratch for the parts while the step runs (see parts/linear.py: a norm handed over between products)
        self.handover = None
        self.upcoming_norm = None
        self.norm_after_block = None

    def attention_work(self, group: int, rows: int, more_than: int = 0):
        """Work list for attention kernels that tile (token, head-in-group) pairs
        in tiles of ``rows``: arrays (request, first pair) and their count.  With
        ``more_than`` only requests that bring more pairs than that are listed."""
        key = (group, rows, more_than)
        if key not in self._work:
            req, pair0 = [], []
            for r, q_len in enumerate(self.host["q_lens"]):
                if q_len * group <= more_than:
                    continue
                for p in range(0, q_len * group, rows):
                    req.append(r)
                    pair0.append(p)
            n = len(req)
            dev = self.rt.staging.upload(np.asarray(req + pair0, dtype=np.int32)) if n else None
            self._work[key] = (dev[:n], dev[n:], n) if n else (None, None, 0)
        return self._work[key]

    def keys_of_small_requests(self, group: int, at_most: int) -> tuple[int, int]:
        """(how many requests bring at most ``at_most`` (token, head-in-group) pairs, the most keys one of them
        holds after this step); needs the host's copy of the step."""
        key = ("small", group, at_most)          # every layer asks; the answer is the step's
        if key in self._work:
            return self._work[key]
        n, keys = 0, 0
        q_lens, before = self.host["q_lens"], self.host.get("ctx_before")
        if before is None:
            return 0, 0
        for q_len, b in zip(q_lens, before):
            if q_len * group <= at_most:
                n += 1
                keys = max(keys, b + q_len)
        self._work[key] = (n, keys)
        return n, keys


def build_context(rt, manager, entries: list[StepEntry]) -> StepContext:
    """Lay a step out for the device.  Pages for the new tokens must be reserved
    already (``manager.reserve``); lengths are advanced by the caller afterwards."""
    ctx = StepContext(rt, manager.page_size)
    ps = manager.page_size
    token_ids, positions, q_start, ctx_before, slots, logit_rows, q_lens = [], [], [0], [], [], [], []
    for e in entries:
        if not e.tokens:
            raise ValueError(f"request {e.rid!r} brings no tokens to the step")
        base = manager.lengths[e.rid]
        n = len(e.tokens)
        for w in e.want:
            if not 0 <= w < n:
                raise ValueError(f"request {e.rid!r}: wanted place {w} is outside its {n} tokens")
            logit_rows.append(len(token_ids) + w)
        token_ids.extend(e.tokens)
        positions.extend(range(base, base + n))
        ctx_before.append(base)
        slots.append(manager.slots[e.rid])
        q_lens.append(n)
        q_start.append(len(token_ids))
    N, R, M = len(token_ids), len(entries), len(logit_rows)
    parts = [token_ids, positions, q_start, ctx_before, slots, logit_rows]
    widths = []
    for g in manager.kv_groups:
        width = max(len(g.tables[e.rid]) for e in entries)
        widths.append(width)
        slot_map = []
        table = np.full((R, width), -1, dtype=np.int32)
        for r, e in enumerate(entries):
            t = g.tables[e.rid]
            table[r, :len(t)] = t
            base = ctx_before[r]
            for p in range(base, base + q_lens[r]):
                page = t[p // ps]
                if page < 0:
                    raise RuntimeError(f"request {e.rid!r}: position {p} lies on a released page")
                slot_map.append(page * ps + p % ps)
        parts.append(slot_map)
        parts.append(table.reshape(-1))
    flat = np.concatenate([np.asarray(p, dtype=np.int32).reshape(-1) for p in parts])
    dev = rt.staging.upload(flat)
    off = 0

    def cut(n):
        nonlocal off
        out = dev[off:off + n]
        off += n
        return out

    ctx.token_ids, ctx.positions, ctx.q_start = cut(N), cut(N), cut(R + 1)
    ctx.ctx_before, ctx.slots, ctx.logit_rows = cut(R), cut(R), cut(M)
    for width in widths:
        sm = cut(N)
        bt = cut(R * width).view(R, width)
        ctx.kv.append(KVGroupContext(sm, bt))
    ctx.n_tokens, ctx.n_requests, ctx.n_logits = N, R, M
    ctx.host = {"token_ids": token_ids, "positions": positions, "q_start": q_start, "ctx_before": ctx_before,
                "slots": slots, "logit_rows": logit_rows, "q_lens": q_lens, "rids": [e.rid for e in entries]}
    ctx.max_q_len = max(q_lens)
    ctx.max_seq_len = max(b + q for b, q in zip(ctx_before, q_lens))
    ctx.keys_cap = ctx.max_seq_len
    return ctx
