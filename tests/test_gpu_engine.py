"""The step function, the cache and generation, in process: long decoding, the
first tokens of a sequence, weights made so that a wrong page or a wrong key
shows, reused pages that hold stale data, greedy and sampled generation through
the Python entry point and the command line."""

import dataclasses
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_llama
from helpers import BF16_NEAR_TIE, TINY, assert_close, make_model_dir, plain_inputs, random_tokens

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def runner_for(model_dir, dtype, **kw):
    from inf_engine_b200 import ModelRunner
    return ModelRunner.from_dir(model_dir, dtype=dtype, **kw)


def entry(rid, toks, want="all"):
    from inf_engine_b200 import StepEntry
    return StepEntry(rid, toks, list(range(len(toks))) if want == "all" else want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_d", "tiny_e", "tiny_f", "tiny_g"])
def test_long_decoding(tmp_path, name, dtype):
    d = make_model_dir(tmp_path, name)
    config, weights = plain_inputs(d)
    toks = random_tokens(config["vocab_size"], 330, 5)
    ref = plain_llama.forward_logits(weights, config, toks)
    r = runner_for(d, dtype, page_size=8, n_pages=48)
    r.open("x")
    rows = [r.step([entry("x", toks[:6])]).cpu().clone()]
    for p in range(6, len(toks)):
        rows.append(r.step([entry("x", toks[p:p + 1])]).cpu().clone())
    assert_close(torch.cat(rows), ref, dtype, f"{name} {dtype} long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_e", "tiny_f", "tiny_g"])
def test_first_tokens_of_a_sequence(tmp_path, name, dtype):
    d = make_model_dir(tmp_path, name)
    config, weights = plain_inputs(d)
    r = runner_for(d, dtype, page_size=16, n_pages=8)
    for n in (1, 2, 3, 17):
        toks = random_tokens(config["vocab_size"], n, 40 + n)
        ref = plain_llama.forward_logits(weights, config, toks)
        r.open("whole")
        assert_close(r.step([entry("whole", toks)]).cpu(), ref, dtype, f"{name} first {n} tokens at once")
        r.close("whole")
        r.open("single")
        rows = [r.step([entry("single", [t])]).cpu().clone() for t in toks]
        assert_close(torch.cat(rows), ref, dtype, f"{name} first {n} tokens one by one")
        r.close("single")


def sharpened(tmp_path, name, factor=5.0):
    """A copy of a tiny model whose q and k projections are scaled up: the softmax becomes
    peaked, each query leans on a few keys far back, and a key read from a wrong page or a
    wrong offset moves the logits far beyond rounding."""
    from inf_engine_b200.weights import open_checkpoint, write_safetensors

    src = make_model_dir(tmp_path, name)
    dst = Path(tmp_path) / f"{name}_sharp"
    dst.mkdir(exist_ok=True)
    t = {k: v.read().clone() for k, v in open_checkpoint(src).items()}
    for k in t:
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            t[k] = (t[k].float() * factor).to(t[k].dtype)
    write_safetensors(dst / "model.safetensors", t)
    (dst / "config.json").write_text((src / "config.json").read_text())
    return dst


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_d", "tiny_e"])
def test_peaked_attention_over_reused_pages(tmp_path, name, dtype):
    # bfloat16 rounds q and k to 8 bits, and a score of size s then carries an error of about
    # s/256 into the exponent: the scores are made 25 times larger in 32-bit, 6 times in bfloat16
    d = sharpened(tmp_path, name, factor=5.0 if dtype == "float32" else 2.5)
    config, weights = plain_inputs(d)
    vocab = config["vocab_size"]
    a, b, c = (random_tokens(vocab, n, s) for n, s in ((300, 1), (170, 2), (260, 3)))
    ref = {k: plain_llama.forward_logits(weights, config, v) for k, v in (("a", a), ("b", b), ("c", c))}
    r = runner_for(d, dtype, page_size=8, n_pages=-(-300 // 8) + -(-170 // 8) + 2)
    got = {"a": [], "b": [], "c": []}
    r.open("a"); r.open("b")
    pa = pb = 0
    while pa < len(a) or pb < len(b):
        es = []
        if pa < len(a):
            n = min(37, len(a) - pa); es.append(entry("a", a[pa:pa + n])); pa += n
        if pb < len(b):
            n = 1 if pb > 150 else min(29, len(b) - pb); es.append(entry("b", b[pb:pb + n])); pb += n
        lg = r.step(es).cpu()
        o = 0
        for e in es:
            got[e.rid].append(lg[o:o + len(e.tokens)].clone()); o += len(e.tokens)
    r.close("a")                                   # c now takes pages that a held; they still hold a's keys
    r.open("c")
    pc = 0
    while pc < len(c):
        n = min(2 + pc % 23, len(c) - pc)
        got["c"].append(r.step([entry("c", c[pc:pc + n])]).cpu().clone()); pc += n
    # the scores of the bfloat16 run are 2.5 x 2.5 times larger, and their rounding error with them: a key from a
    # wrong page or offset moves the logits by their own size, a hundred times this bound
    for k in got:
        assert_close(torch.cat(got[k]), ref[k], dtype, f"{name} {dtype} peaked request {k}", noise=2.5)
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_model_with_a_window_layer_a_shared_cache_and_a_layer_run_twice(tmp_path, dtype):
    """The order of layers is data: layer 0 (full attention), then layer 1 (a window of 24)
    run twice, each run with a cache of its own, then layer 2 reading layer 0's cache.
    Checked against the plain functions put together the same way."""
    from inf_engine_b200 import ModelRunner
    from inf_engine_b200.config import ScheduleEntry, parse_config_dict
    from inf_engine_b200.parts import expected_tensors
    from inf_engine_b200.weights import load_weights

    name = "tiny_b"
    d = make_model_dir(tmp_path, name)
    config, weights = plain_inputs(d)
    cfg = parse_config_dict(TINY[name])
    base = cfg.model_spec()
    window = 24
    layers = list(base.layers)
    layers[1] = dataclasses.replace(layers[1], mixer=dataclasses.replace(layers[1].mixer, window=window))
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(2, cache_from=0))
    spec = dataclasses.replace(base, layers=tuple(layers), schedule=schedule)
    run_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = load_weights(d, expected_tensors(spec), run_dtype, "cuda:0")
    r = ModelRunner(cfg, tensors, run_dtype, page_size=8, n_pages=40, spec=spec)
    assert len(r.cache.kv_groups) == 2 and r.cache.kv_groups[1].window == window
    assert len(r.cache.kv_groups[1].entries) == 2               # layer 1's two runs have a cache each

    toks = random_tokens(config["vocab_size"], 150, 9)

    def plain_forward(toks):
        w = weights
        T = len(toks)
        x = w["model.embed_tokens.weight"][torch.tensor(toks)]
        cos, sin = plain_llama.rope_tables(config, T)
        eps = config["rms_norm_eps"]
        kv0 = None
        for run, (layer, win, shared) in enumerate([(0, None, False), (1, window, False), (1, window, False), (2, None, True)]):
            p = f"model.layers.{layer}."
            h = plain_llama.rms_norm(x, w[p + "input_layernorm.weight"], eps)
            wk, wv = w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"]
            if run == 0:
                kv0 = h
            if shared:
                # keys and values come from the cache of run 0: layer 0's projections of layer 0's input
                p0 = "model.layers.0."
                att = _attention_with_foreign_kv(h, kv0, w[p + "self_attn.q_proj.weight"],
                                                 w[p0 + "self_attn.k_proj.weight"], w[p0 + "self_attn.v_proj.weight"],
                                                 w[p + "self_attn.o_proj.weight"], config, cos, sin)
            else:
                att = plain_llama.attention(h, w[p + "self_attn.q_proj.weight"], wk, wv,
                                            w[p + "self_attn.o_proj.weight"], config, cos, sin, window=win)
            x = x + att
            h = plain_llama.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
            x = x + plain_llama.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        x = plain_llama.rms_norm(x, w["model.norm.weight"], eps)
        return x @ w["lm_head.weight"].T

    ref = plain_forward(toks)
    r.open("x")
    rows, p = [], 0
    for n in [31, 2, 40, 1, 1, 1, 17, 57]:
        rows.append(r.step([entry("x", toks[p:p + n])]).cpu().clone()); p += n
        r.cache.check()
    assert p == len(toks)
    assert_close(torch.cat(rows), ref, dtype, f"window/shared/twice {dtype}")
    # the window group gave pages back as it moved; the full group kept all
    assert r.cache.kv_groups[1].pool.n_held <= -(-window // 8) + 1
    assert r.cache.kv_groups[0].pool.n_held == -(-150 // 8)


def _attention_with_foreign_kv(h_q, h_kv, wq, wk, wv, wo, config, cos, sin):
    """plain_llama.attention with keys and values projected from another run's input."""
    T = h_q.shape[0]
    H, Hk, hd = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    q = (h_q @ wq.T).view(T, H, hd).transpose(0, 1)
    k = (h_kv @ wk.T).view(T, Hk, hd).transpose(0, 1)
    v = (h_kv @ wv.T).view(T, Hk, hd).transpose(0, 1)
    q, k = plain_llama.apply_rope(q, cos[:T], sin[:T]), plain_llama.apply_rope(k, cos[:T], sin[:T])
    g = H // Hk
    k = k[:, None].expand(Hk, g, T, hd).reshape(H, T, hd)
    v = v[:, None].expand(Hk, g, T, hd).reshape(H, T, hd)
    s = (q @ k.transpose(1, 2)) * hd ** -0.5
    s = s.masked_fill(~(torch.arange(T)[None, :] <= torch.arange(T)[:, None])[None], float("-inf"))
    return (torch.softmax(s, -1) @ v).transpose(0, 1).reshape(T, H * hd) @ wo.T


def test_step_refuses_what_it_cannot_run(tmp_path):
    from inf_engine_b200 import OutOfPages
    d = make_model_dir(tmp_path, "tiny_a")
    r = runner_for(d, "float32", page_size=16, n_pages=2)
    r.open("x")
    with pytest.raises(ValueError, match="vocabulary"):
        r.step([entry("x", [1, 999])])
    with pytest.raises(OutOfPages):
        r.step([entry("x", list(range(40)))])
    assert r.cache.n_free_pages() == 2 and r.length("x") == 0      # nothing taken
    with pytest.raises(KeyError):
        r.step([entry("nobody", [1])])
    with pytest.raises(ValueError, match="twice"):
        r.step([entry("x", [1]), entry("x", [2])])
    assert r.step([entry("x", [1, 2, 3], want=[])]) is None           # nothing wanted: nothing returned


# ------------------------------------------------------------------- generation
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_d"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    from inf_engine_b200 import Engine, Request
    d = make_model_dir(tmp_path, name)
    config, weights = plain_inputs(d)
    vocab = config["vocab_size"]
    prompts = [random_tokens(vocab, n, 60 + n) for n in (5, 17, 33, 1)]
    engine = Engine.from_dir(d, dtype=dtype, n_total_blocks=24, block_size=8, max_tokens_per_step=24, chunk=16)
    out = engine.run_offline([Request(i, p, max_new_tokens=8) for i, p in enumerate(prompts)])
    for i, p in enumerate(prompts):
        got = out[i]
        assert len(got) == 8
        # every generated token is the plain implementation's choice given the same prefix
        # (in bfloat16: a token whose plain logit is within rounding of the best)
        logits = plain_llama.forward_logits(weights, config, p + got)
        for j, tok in enumerate(got):
            row = logits[len(p) + j - 1]
            if dtype == "float32":
                assert tok == int(row.argmax()), f"{name} request {i} token {j}"
            else:
                assert float(row.max() - row[tok]) <= BF16_NEAR_TIE * max(1.0, float(row.abs().max()))
    assert engine.runner.cache.n_free_pages() == 24 and engine.stats["prefill_tokens"] >= 56
    if dtype == "float32":
        assert out[0] == plain_llama.greedy_generate(weights, config, prompts[0], 8)


@pytest.mark.parametrize("name,dtype", [("tiny_a", "float32"), ("tiny_d", "bfloat16")])
def test_graphs_follow_the_growing_context_and_old_ones_are_dropped(tmp_path, monkeypatch, name, dtype):
    """Decode graphs are captured per step of the longest context; with a step of 8 keys and room for two
    graphs, 40 generated tokens go through many captures and evictions and still equal the plain choice."""
    from inf_engine_b200 import Engine, Request
    from inf_engine_b200.engine import graphs
    monkeypatch.setattr(graphs, "KEYS_STEP", 8)
    monkeypatch.setattr(graphs, "MAX_GRAPHS", 2)
    d = make_model_dir(tmp_path, name)
    config, weights = plain_inputs(d)
    prompts = [random_tokens(config["vocab_size"], n, 70 + n) for n in (3, 11)]
    engine = Engine.from_dir(d, dtype=dtype, n_total_blocks=32, block_size=8)
    out = engine.run_offline([Request(i, p, max_new_tokens=40) for i, p in enumerate(prompts)])
    g = engine.runner.graphs
    assert g.captures >= 5 and len(g._buckets) <= 2
    for i, p in enumerate(prompts):
        logits = plain_llama.forward_logits(weights, config, p + out[i])
        for j, tok in enumerate(out[i]):
            row = logits[len(p) + j - 1]
            if dtype == "float32":
                assert tok == int(row.argmax())
            else:
                assert float(row.max() - row[tok]) <= BF16_NEAR_TIE * max(1.0, float(row.abs().max()))


def test_generation_survives_a_pool_that_runs_out(tmp_path):
    """Pages run out while decoding: the youngest request is preempted and recomputed;
    every request still gets exactly the tokens it gets when it runs alone."""
    from inf_engine_b200 import Engine, Request
    d = make_model_dir(tmp_path, "tiny_a")
    config, _ = plain_inputs(d)
    prompts = [random_tokens(config["vocab_size"], n, 80 + n) for n in (30, 21, 26, 9)]
    alone = Engine.from_dir(d, dtype="float32", n_total_blocks=64, block_size=4)
    want = [alone.generate(p, 40) for p in prompts]
    tight = Engine.from_dir(d, dtype="float32", n_total_blocks=40, block_size=4, max_tokens_per_step=32)
    out = tight.run_offline([Request(i, p, max_new_tokens=40) for i, p in enumerate(prompts)])
    assert tight.stats["preemptions"] >= 1
    assert [out[i] for i in range(4)] == want
    tight.runner.cache.check()
    assert tight.runner.cache.n_free_pages() == 40


def test_sampled_generation_is_seeded_and_independent_of_the_batch(tmp_path):
    from inf_engine_b200 import Engine, Request, SamplingConfig
    d = make_model_dir(tmp_path, "tiny_b")
    config, weights = plain_inputs(d)
    prompts = [random_tokens(config["vocab_size"], n, 90 + n) for n in (1, 9, 40, 70)]
    s = SamplingConfig(mode="temperature", temperature=0.7, seed=1)
    e1 = Engine.from_dir(d, dtype="float32", n_total_blocks=64, block_size=8, max_tokens_per_step=64, chunk=16)
    batch = e1.run_offline([Request(i, p, 12, sampling=s) for i, p in enumerate(prompts)])
    e2 = Engine.from_dir(d, dtype="float32", n_total_blocks=64, block_size=8)
    for i, p in enumerate(prompts):
        assert e2.generate(p, 12, sampling=s, req_id=i) == batch[i]
    other = e2.generate(prompts[2], 12, sampling=SamplingConfig(mode="temperature", temperature=0.7, seed=2), req_id=2)
    assert other != batch[2]
    # with random weights the distribution is nearly flat: sampling does not repeat the greedy answer
    assert batch[2] != e2.generate(prompts[2], 12, req_id=2)
    # stop at EOS: the token is kept and the request ends (engine/llama_paged_engine.py:207-211)
    eos = batch[3][4]
    e3 = Engine.from_dir(d, dtype="float32", n_total_blocks=64, block_size=8, eos_token=eos)
    got = e3.run_offline([Request(3, prompts[3], 12, sampling=s)])[3]
    assert got == batch[3][:batch[3].index(eos) + 1]


@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_enqueued_one_ahead_give_the_same_tokens(tmp_path, dtype):
    """With ``pipeline`` a step is enqueued before the tokens of the step before are read; requests that end
    by their token (EOS, stop_check) are found out one step late and the extra step is dropped."""
    from inf_engine_b200 import Engine, Request, SamplingConfig
    d = make_model_dir(tmp_path, "tiny_b")
    config, _ = plain_inputs(d)
    prompts = [random_tokens(config["vocab_size"], n, 70 + n) for n in (3, 30, 11, 50, 7)]
    s = SamplingConfig(mode="top_p", top_p=0.95, temperature=0.9, seed=11)

    def run(pipeline, eos=None, stop=None):
        e = Engine.from_dir(d, dtype=dtype, n_total_blocks=64, block_size=8, max_tokens_per_step=48, chunk=16,
                            eos_token=eos, pipeline=pipeline)
        reqs = [Request(i, p, 14 + i, sampling=s, stop_check=stop if i == 1 else None) for i, p in enumerate(prompts)]
        out = e.run_offline(reqs)
        e.runner.cache.check()
        assert e.runner.cache.n_free_pages() == 64 and not e.has_work
        return [out[i] for i in range(len(prompts))]

    base = run(False)
    assert run(True) == base
    assert all(t >= 0 for g in base for t in g)
    eos = base[3][5]                                           # a token that request 3 produces mid-way
    stop = lambda g: len(g) >= 4
    a, b = run(False, eos, stop), run(True, eos, stop)
    assert a == b and len(a[1]) == 4
    assert a[3] == base[3][:base[3].index(eos) + 1]


def test_command_line(tmp_path):
    d = make_model_dir(tmp_path, "tiny_a")
    config, weights = plain_inputs(d)
    root = Path(__file__).resolve().parent.parent
    stats = tmp_path / "stats.json"
    p = subprocess.run([sys.executable, str(root / "bin" / "generate_llama"), "--model-dir", str(d), "--dtype", "float32",
                        "--prompt-ids", "5,17,3;9,9,9,9", "--n", "6", "--stats-json", str(stats),
                        "--trace-jsonl", str(tmp_path / "steps.jsonl"), "--nvtx"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if ":" in l]
    got = {int(l.split(":")[0]): [int(t) for t in l.split(":")[1].split(",")] for l in lines}
    assert got[0] == plain_llama.greedy_generate(weights, config, [5, 17, 3], 6)
    assert got[1] == plain_llama.greedy_generate(weights, config, [9, 9, 9, 9], 6)
    st = json.loads(stats.read_text())
    assert st["new_tokens"] == 12
    # time to the first token and time per later token, per request and summed up
    assert len(st["requests"]) == 2 and all(r["ttft_s"] > 0 and r["tpot_s"] > 0 for r in st["requests"])
    assert 0 < st["ttft_s"]["p50"] <= st["ttft_s"]["max"] and st["tpot_s"]["mean"] > 0
    # one line per step: the first step holds both prompts, the later ones a decoded token of each
    steps = [json.loads(l) for l in (tmp_path / "steps.jsonl").read_text().splitlines()]
    assert len(steps) == st["steps"] and steps[0]["prefill_tokens"] == 7 and steps[0]["requests"] == 2
    assert sum(s["prefill_tokens"] + s["decode_tokens"] for s in steps) == st["prefill_tokens"] + st["decode_tokens"]
    assert all(s["host_us"] > 0 and s["pages_free"] >= 0 for s in steps) and steps[-1]["decode_tokens"] >= 1


@pytest.mark.parametrize("preset,layers", [("llama-3.2-1b", 2), ("llama-3.2-3b", 1), ("smollm2-1.7b", 2)])
def test_full_width_layers_against_the_plain_implementation(tmp_path, preset, layers):
    """The real widths (hidden 2,048 / 3,072, heads of 64 / 128, grouped and not, vocabularies of 128,256 and 49,152)
    take the kernels' large-size paths, which most tiny models never reach: the tensor-core products and attention of
    a long prompt, the streaming products with the norm handed over and the split-key attention of decode steps
    inside captured graphs, and a mixed step.  Both precisions against the plain implementation, whose head runs on
    the wanted rows only (engine/llama_model.py:147-148 computes every row's)."""
    from inf_engine_b200.config import get_preset
    from inf_engine_b200.weights import write_random_model

    cfg = dataclasses.replace(get_preset(preset), num_hidden_layers=layers)
    d = tmp_path / "wide"
    write_random_model(cfg, 11, d)
    config, weights = plain_inputs(d)
    V = cfg.vocab_size
    a, b = random_tokens(V, 300, 1), random_tokens(V, 150, 2)
    tail = random_tokens(V, 4, 3)
    a_all, b_all = a + tail + [7, 8], b + [8, 9]
    # (request, position) of every row the steps below ask for, in order
    asked = [("a", 298), ("a", 299), ("a", 300), ("a", 301), ("a", 302), ("b", 99), ("a", 303), ("b", 149),
             ("a", 304), ("b", 150), ("a", 305), ("b", 151)]
    ref_a = plain_llama.forward_logits(weights, config, a_all, rows=[p for r, p in asked if r == "a"])
    ref_b = plain_llama.forward_logits(weights, config, b_all, rows=[p for r, p in asked if r == "b"])
    ia = ib = 0
    ref = []
    for r, _ in asked:
        if r == "a":
            ref.append(ref_a[ia]); ia += 1
        else:
            ref.append(ref_b[ib]); ib += 1
    ref = torch.stack(ref)
    del weights

    def run(dtype):
        r = runner_for(d, dtype, page_size=16, n_pages=64, max_requests=4)
        out = []
        r.open("a")
        out.append(r.step([entry("a", a, [len(a) - 2, len(a) - 1])]).cpu().clone())       # a long prompt, whole
        for t in tail[:2]:                                                                 # decode steps of one
            out.append(r.step([entry("a", [t])]).cpu().clone())
        r.open("b")
        out.append(r.step([entry("a", [tail[2]]), entry("b", b[:100], [99])]).cpu().clone())   # mixed
        out.append(r.step([entry("a", [tail[3]]), entry("b", b[100:], [49])]).cpu().clone())
        for t in (7, 8):                                                                   # decode steps of two
            out.append(r.step([entry("a", [t]), entry("b", [t + 1])]).cpu().clone())
        return torch.cat(out)

    assert_close(run("float32"), ref, "float32", f"{preset} widths, {layers} layers, float32")
    assert_close(run("bfloat16"), ref, "bfloat16", f"{preset} widths, {layers} layers, bfloat16")


def test_preset_tiny_b_sampled_workload_follows_the_plain_distribution(tmp_path):
    """The tiny-b preset exactly as stated (3 layers, one kv head for four query heads, llama3 scaling, pages of 8):
    prompts of 1, 9, 40 and 70 tokens as a mixed batch in portions of 16, then 12 tokens each at temperature 0.7,
    seed 1.  Every token the engine draws must be the one the plain implementation's distribution gives at the
    number hashed from (seed, request, how many it had generated): plain logits, temperature, softmax, inverse CDF."""
    from inf_engine_b200 import Engine, Request, SamplingConfig
    from inf_engine_b200.sampling import request_key, uniform_of

    d = make_model_dir(tmp_path, "tiny-b")
    config, weights = plain_inputs(d)
    assert (config["num_hidden_layers"], config["num_key_value_heads"], config["head_dim"], config["vocab_size"]) == (3, 1, 32, 384)
    prompts = [random_tokens(config["vocab_size"], n, 90 + n) for n in (1, 9, 40, 70)]
    s = SamplingConfig(mode="temperature", temperature=0.7, seed=1)
    for pipeline in (False, True):
        engine = Engine.from_dir(d, dtype="float32", n_total_blocks=64, block_size=8, max_tokens_per_step=64, chunk=16,
                                 pipeline=pipeline)
        out = engine.run_offline([Request(i, p, 12, sampling=s) for i, p in enumerate(prompts)])
        for i, p in enumerate(prompts):
            assert len(out[i]) == 12
            logits = plain_llama.forward_logits(weights, config, p + out[i])
            for j, tok in enumerate(out[i]):
                probs = plain_llama.filtered_distribution(logits[len(p) + j - 1], "temperature", temperature=0.7).double()
                cdf = probs.cumsum(0)
                u = uniform_of(1, request_key(i, j))
                lo = float(cdf[tok - 1]) if tok > 0 else 0.0
                assert lo - 2e-5 <= u <= float(cdf[tok]) + 2e-5, \
                    f"request {i} token {j}: u={u} is outside [{lo}, {float(cdf[tok])}] of token {tok}"


def test_preset_tiny_a_workload_is_the_plain_greedy_continuation(tmp_path):
    """The tiny-a preset exactly as stated: prompts of 5, 17 and 33 tokens, 8 greedy tokens each, pages of 16."""
    from inf_engine_b200 import Engine, Request

    d = make_model_dir(tmp_path, "tiny-a")
    config, weights = plain_inputs(d)
    prompts = [random_tokens(config["vocab_size"], n, 50 + n) for n in (5, 17, 33)]
    engine = Engine.from_dir(d, dtype="float32", n_total_blocks=16, block_size=16)
    out = engine.run_offline([Request(i, p, 8) for i, p in enumerate(prompts)])
    for i, p in enumerate(prompts):
        assert out[i] == plain_llama.greedy_generate(weights, config, p, 8)
