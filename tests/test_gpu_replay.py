"""Trace replay through ``bin/trace_run`` as a user runs it, compared with the
plain implementation: each request alone and whole; most of it in one step and
the last 32 tokens one by one; in portions of changing size down to two tokens;
and mixed, up to four live requests, portions of some beside decoded tokens of
others, in a pool so small that pages are used again.  In 32-bit and bfloat16."""

import random

import pytest
import torch

import plain_llama
from helpers import TINY, TraceBuilder, assert_close, make_model_dir, plain_inputs, random_tokens, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [70, 45, 130, 20, 97, 33, 150], "tiny_b": [64, 129, 40, 200, 31, 16, 77],
           "tiny_d": [81, 300, 47, 160, 33, 210, 65], "tiny_e": [150, 66, 260, 40, 129, 90, 35],
           "tiny_f": [90, 280, 47, 170, 33, 140, 65], "tiny_g": [300, 70, 150, 45, 33, 190, 64],
           "tiny-a": [5, 17, 33, 100, 128, 90, 64, 120], "tiny-b": [1, 9, 40, 70, 129, 200, 64, 250, 180]}
PAGE = {"tiny_a": 16, "tiny_b": 8, "tiny_d": 16, "tiny_e": 32, "tiny_f": 16, "tiny_g": 16, "tiny-a": 16, "tiny-b": 8}
NAMES = ["tiny_a", "tiny_b", "tiny_d", "tiny_e", "tiny_f", "tiny_g", "tiny-a", "tiny-b"]


def schedules(name: str, requests: dict[str, list[int]], seed: int) -> TraceBuilder:
    rng = random.Random(seed)
    t = TraceBuilder()
    ids = list(requests)
    # (1) each request alone and whole
    for rid in ids[:3]:
        t.step([("w" + rid, requests[rid], 0)], end=["w" + rid])
    # (2) most of it in one step, the last 32 tokens one by one
    for rid in ids[:2]:
        toks = requests[rid]
        cut = max(len(toks) - 32, 1)
        t.step([("d" + rid, toks[:cut], 0)])
        for p in range(cut, len(toks)):
            t.step([("d" + rid, toks[p:p + 1], p)], end=["d" + rid] if p == len(toks) - 1 else [])
    # (3) portions of changing size, down to two tokens
    for rid in ids[2:4]:
        toks, p = requests[rid], 0
        sizes = [7, 2, 16, 3, 2, 17, 2, 31, 1, 5]
        i = 0
        while p < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - p)
            t.step([("p" + rid, toks[p:p + n], p)], end=["p" + rid] if p + n == len(toks) else [])
            p += n
            i += 1
    # (4) mixed: up to four live, portions beside decoded tokens, some left out of a step
    waiting = [("m" + rid, requests[rid]) for rid in ids]
    live: dict[str, list] = {}
    while waiting or live:
        while waiting and len(live) < 4:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, max(1, len(toks) - rng.choice([3, 9, 20]))]   # tokens, done, where decoding starts
        entries, ended = [], []
        for rid, st in list(live.items()):
            toks, done, decode_from = st
            if rng.random() < 0.2 and len(live) > 1:
                continue                                                      # left out of this step
            n = 1 if done >= decode_from else min(rng.choice([2, 3, 5, 11, 17, 40]), decode_from - done)
            entries.append((rid, toks[done:done + n], done))
            st[1] = done + n
            if st[1] == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            t.step(entries, end=ended)
    return t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_replay_under_every_cut(tmp_path, name, dtype):
    model_dir = make_model_dir(tmp_path, name)
    config, weights = plain_inputs(model_dir)
    vocab = config["vocab_size"]
    requests = {str(i): random_tokens(vocab, n, 100 + i) for i, n in enumerate(LENGTHS[name])}
    trace = schedules(name, requests, seed=len(name) + NAMES.index(name))
    # the pool is exactly what the trace holds at its fullest, so pages of finished requests are used again
    assert trace.max_tokens < sum(len(v) for v in requests.values())
    got = run_trace(model_dir, dtype, trace, tmp_path / "out", vocab, page_size=PAGE[name])
    plain = {rid: plain_llama.forward_logits(weights, config, toks) for rid, toks in requests.items()}
    by_request: dict[str, list] = {}
    for (rid, pos), row in got.items():
        by_request.setdefault(rid, []).append((pos, row))
    assert len(by_request) == 3 + 2 + 2 + len(requests)
    for rid, rows in by_request.items():
        rows.sort(key=lambda x: x[0])
        ref = plain[rid[1:]]
        assert [p for p, _ in rows] == list(range(ref.shape[0])), f"{rid}: positions missing"
        assert_close(torch.stack([r for _, r in rows]), ref, dtype, what=f"{name} {dtype} request {rid}")
    if dtype == "float32":
        # in 32-bit the cuts agree with each other far below the tolerance against the plain implementation
        for rid in list(requests)[:2]:
            if len(requests[rid]) < 2:
                continue
            whole = torch.stack([got[("w" + rid, p)] for p in range(len(requests[rid]))])
            cut = torch.stack([got[("d" + rid, p)] for p in range(len(requests[rid]))])
            mixed = torch.stack([got[("m" + rid, p)] for p in range(len(requests[rid]))])
            assert float((whole - cut).abs().max()) < 1e-6 and float((whole - mixed).abs().max()) < 1e-6


def many_live_schedule(requests: dict[str, list[int]], seed: int) -> TraceBuilder:
    """Up to 36 requests live at once: waves of prompts (whole or in portions) beside the decoded tokens of
    everybody else, then runs of steps in which 20 to 36 requests decode together, some leaving and new ones
    joining in between.  More than 16 rows in a decode step take other kernels than the few-row steps do."""
    rng = random.Random(seed)
    t = TraceBuilder()
    waiting = list(requests.items())
    live: dict[str, list] = {}            # rid -> [tokens, done, where decoding starts]

    def step(only_decoding: bool):
        entries, ended = [], []
        for rid, st in list(live.items()):
            toks, done, decode_from = st
            if done < decode_from:
                n = min(rng.choice([2, 5, 13, 24]), decode_from - done)
            elif only_decoding or rng.random() < 0.9:
                n = 1
            else:
                continue
            entries.append((rid, toks[done:done + n], done))
            st[1] = done + n
            if st[1] == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            t.step(entries, end=ended)

    def admit(n: int, tail: tuple[int, int]):
        for _ in range(min(n, len(waiting))):
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0, max(1, len(toks) - rng.randint(*tail))]

    admit(28, (44, 52))
    while any(st[1] < st[2] for st in live.values()):
        step(False)                        # prompts in portions, early finishers already decoding beside them
    for _ in range(12):
        step(True)                         # 28 decoding together
    admit(8, (30, 40))
    while any(st[1] < st[2] for st in live.values()):
        step(False)                        # portions of the newcomers beside 28 decoded tokens
    for _ in range(14):
        step(True)                         # 36 decoding together
    admit(len(waiting), (8, 12))
    while live:
        step(False)
    return t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_d", "tiny_f", "tiny_g"])
def test_replay_with_many_requests_decoding_together(tmp_path, name, dtype):
    model_dir = make_model_dir(tmp_path, name)
    config, weights = plain_inputs(model_dir)
    vocab = config["vocab_size"]
    rng = random.Random(7)
    requests = {f"r{i}": random_tokens(vocab, rng.randint(70, 130), 300 + i) for i in range(44)}
    trace = many_live_schedule(requests, seed=3)
    sizes = [len(s["entries"]) for s in trace.steps]
    decode_only = [len(s["entries"]) for s in trace.steps if all(len(e["tokens"]) == 1 for e in s["entries"])]
    assert max(sizes) >= 34 and sum(1 for n in decode_only if n > 16) >= 20 and sum(1 for n in decode_only if n > 32) >= 10
    assert any(any(len(e["tokens"]) > 1 for e in s["entries"]) and sum(len(e["tokens"]) == 1 for e in s["entries"]) > 16
               for s in trace.steps)          # portions beside more than 16 decoded tokens
    got = run_trace(model_dir, dtype, trace, tmp_path / "out", vocab, page_size=PAGE[name])
    by_request: dict[str, list] = {}
    for (rid, pos), row in got.items():
        by_request.setdefault(rid, []).append((pos, row))
    assert set(by_request) == set(requests)
    for rid, rows in by_request.items():
        rows.sort(key=lambda x: x[0])
        ref = plain_llama.forward_logits(weights, config, requests[rid])
        assert [p for p, _ in rows] == list(range(ref.shape[0])), f"{rid}: positions missing"
        assert_close(torch.stack([r for _, r in rows]), ref, dtype, what=f"{name} {dtype} many live, request {rid}")
