"""Benchmark of the engine on one B200: decode tokens per second at batch 8 (and 1
and 64), prefill of one 2,048-token prompt, at Llama-3.2-1B size with random
weights and uniform random prompt ids.

    python bench.py --gpus 1 --steps K --warmup W      -> one JSON line
    python bench.py --impl reference ...               -> the reference arm (or why it is unavailable)

A "step" is one decode step of the whole batch.  ``value`` is device-timed
(CUDA events around K steps fed from the device); ``e2e`` is the same through
``Engine.step`` with host tokens in and out every step.  Weights (2.5 GB) are
larger than L2, so every step streams them from HBM: no L2 flush is needed.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PROMPT_LEN = 2048
POOL_CONTEXT = 4096
PAGE = 16


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, t0, t1):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.samples:
            if not (t0 - 0.05 <= t <= t1 + 0.15):
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                sm.append(int(parts[0]))
                mx = max(mx, int(parts[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def model_numbers(cfg):
    d, L, H, Hk, hd, I, V = (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads,
                             cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size)
    per_layer = (H * hd + 2 * Hk * hd) * d + d * H * hd + 3 * I * d
    linear_params = L * per_layer
    head_params = V * d
    weight_bytes = 2 * (linear_params + head_params) + 2 * 2 * L * d + 2 * d       # bf16; norms are small
    kv_bytes_per_token = 2 * L * Hk * hd * 2
    return dict(linear_params=linear_params, head_params=head_params, weight_bytes=weight_bytes,
                kv_bytes_per_token=kv_bytes_per_token)


def prefill_flops(cfg, n):
    m = model_numbers(cfg)
    attn = cfg.num_hidden_layers * 4 * cfg.num_attention_heads * cfg.head_dim * (n * (n + 1) // 2)
    return 2 * n * m["linear_params"] + attn + 2 * m["head_params"]


def run_ours(args):
    import numpy as np
    import torch

    from inf_engine_b200 import Engine, Request, SamplingConfig, StepEntry, kernels
    from inf_engine_b200.config import get_preset
    from inf_engine_b200.sampling import pack_rows, request_key
    from inf_engine_b200.weights import write_random_model

    cfg = get_preset(args.model)
    n_layers_full = cfg.num_hidden_layers
    if args.layers:
        import dataclasses
        cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers)
    pk = peaks()
    torch.cuda.set_device(0)
    t_build = time.perf_counter()
    with tempfile.TemporaryDirectory(prefix="bench_model_") as tmp:
        write_random_model(cfg, args.seed, tmp)
        engine = Engine.from_dir(tmp, dtype="bfloat16", n_total_blocks=args.pool_requests * POOL_CONTEXT // PAGE, block_size=PAGE,
                                 max_requests=max(64, args.pool_requests), max_tokens_per_step=8192, chunk=2048)
    t_build = time.perf_counter() - t_build
    runner = engine.runner
    V = cfg.vocab_size
    rng = np.random.default_rng(args.seed)
    nums = model_numbers(cfg)
    clocks = ClockSampler()
    clocks.start()

    def prompt():
        return rng.integers(0, V, PROMPT_LEN).tolist()

    # ---------------------------------------------------------------- prefill
    def prefill_once():
        runner.open("p")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        toks = prompt()
        torch.cuda.synchronize()
        e0.record()
        runner.step([StepEntry("p", toks, [PROMPT_LEN - 1])])
        e1.record()
        torch.cuda.synchronize()
        runner.close("p")
        return e0.elapsed_time(e1)

    if args.only == "decode":
        pre_ms = [float("nan")]
    else:
        for _ in range(3):
            prefill_once()
        pre_ms = sorted(prefill_once() for _ in range(args.prefill_reps))
    pre = pre_ms[len(pre_ms) // 2]
    prefill = {"value": PROMPT_LEN / pre * 1e3, "unit": "tok/s", "tokens": PROMPT_LEN, "ms": pre,
               "frac": prefill_flops(cfg, PROMPT_LEN) / (pre * 1e-3) / (pk["bf16_tflops"] * 1e12),
               "peak_tflops": pk["bf16_tflops"], "peak_source": pk["source"]}

    # ----------------------------------------------------------------- decode
    greedy = SamplingConfig()

    def decode_device(batch, steps, warmup):
        """Device-timed decode: K steps, each fed the ids the step before sampled, no host read inside."""
        rids = [f"d{batch}_{i}" for i in range(batch)]
        for rid in rids:
            runner.open(rid)
        for i in range(0, batch, 4):                      # prompts, four at a time
            runner.step([StepEntry(r, prompt(), []) for r in rids[i:i + 4]])
        rows = pack_rows([greedy] * batch, [request_key(i, 0) for i in range(batch)], V)
        ids = torch.as_tensor(rng.integers(0, V, batch), dtype=torch.int32).cuda()
        entries = [StepEntry(r, [0], [0]) for r in rids]
        for _ in range(warmup):
            _, ids = runner.step_and_sample(entries, rows, device_tokens=ids)
        gc.collect()          # a full collection of the host's garbage inside the timed steps would stall the launches
        torch.cuda.synchronize()
        ctx0 = runner.length(rids[0])
        n0 = kernels.LAUNCHES
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            _, ids = runner.step_and_sample(entries, rows, device_tokens=ids)
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        ms = e0.elapsed_time(e1)
        launches = kernels.LAUNCHES - n0
        for rid in rids:
            runner.close(rid)
        mean_ctx = ctx0 + steps / 2
        bytes_step = nums["weight_bytes"] + batch * mean_ctx * nums["kv_bytes_per_token"]
        return dict(tok_s=batch * steps / ms * 1e3, ms_per_step=ms / steps, launches=launches, t0=t0, t1=t1,
                    bytes_step=bytes_step, ctx=(ctx0, ctx0 + steps))

    def decode_e2e(batch, steps, warmup):
        """Through Engine.step: host tokens in (one pinned copy a step), sampled ids out (one read a step)."""
        reqs = [Request(1000 + i, prompt(), max_new_tokens=warmup + steps + 8) for i in range(batch)]
        for r in reqs:
            assert engine.submit(r), r.error
        while any(len(r.generated) < 1 for r in reqs):
            engine.step()
        for _ in range(warmup):
            engine.step()
        gc.collect()
        torch.cuda.synchronize()
        n_before = sum(len(r.generated) for r in reqs)
        t0 = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        n_tok = sum(len(r.generated) for r in reqs) - n_before
        while engine.has_work:
            engine.step()
        engine.completed.clear()
        b = next(iter(runner.graphs._buckets.values()))
        key = [k for k in runner.graphs._buckets if k[0] >= batch]
        h2d = min(runner.graphs._buckets[k].n for k in key) * 4 if key else 0
        return dict(tok_s=n_tok / (t1 - t0), h2d=h2d, d2h=4 * batch)

    if args.only == "prefill":
        clocks.stop()
        print(json.dumps({"impl": "ours", "only": "prefill", "prefill": prefill, "config": {"model": args.model, "layers": cfg.num_hidden_layers}}))
        return 0
    main = decode_device(args.batch, args.steps, args.warmup)
    if args.only == "decode":
        clocks.stop()
        print(json.dumps({"impl": "ours", "only": "decode", "value": main["tok_s"], "ms_per_step": main["ms_per_step"],
                          "config": {"model": args.model, "layers": cfg.num_hidden_layers, "global_batch": args.batch}}))
        return 0
    e2e = decode_e2e(args.batch, args.steps, args.warmup)
    points = {}
    for b in (1, 64):
        if b <= args.pool_requests:
            points[f"decode_b{b}"] = decode_device(b, args.steps, args.warmup)["tok_s"]
    clocks.stop()
    clk = clocks.summary(main["t0"], main["t1"])
    # the other two configurations of the baseline: continuous batching at their sizes, wall clock
    workloads = {}
    if not args.no_workloads:
        del engine, runner
        gc.collect()
        torch.cuda.empty_cache()
        for key, model, n_req, lo, hi, new, temps in WORKLOADS:
            for rec in measure_workload(model, n_req, lo, hi, new, temps, args.seed):
                workloads[key + ("" if rec["temperature"] == 0 else f"_t{rec['temperature']}")] = {
                    k: rec[k] for k in ("seconds", "generated_tok_s", "total_tok_s", "steps", "preemptions",
                                        "ttft_s_p50", "tpot_s_mean")}

    achieved = main["bytes_step"] / (main["ms_per_step"] * 1e-3) / 1e9
    out = {
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B size, random weights)",
        "value": main["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random prompt ids", "impl": "ours",
        "config": {
            "model": args.model, "layers": cfg.num_hidden_layers, "layers_of_model": n_layers_full,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "seq_len": PROMPT_LEN, "context_start": main["ctx"][0],
            "context_end": main["ctx"][1], "pool_context": POOL_CONTEXT, "page_size": PAGE,
            "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights 2.5 GB per step)",
            "decode": "cuda graph per batch bucket, sampling in graph",
        },
        "e2e": {"value": e2e["tok_s"], "unit": "tok/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": main["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"]},
        "points": points,
        "workloads": workloads,
        "clocks": clk,
        "build_s": t_build,
    }
    print(json.dumps(out))
    return 0


# BASELINE.json's other two configurations: (key, preset, requests, shortest and longest prompt, new tokens, temperatures)
WORKLOADS = [("llama-3.2-3b_32req_128-4096_128new", "llama-3.2-3b", 32, 128, 4096, 128, (0.0,)),
             ("smollm2-1.7b_64req_64-2048_256new", "smollm2-1.7b", 64, 64, 2048, 256, (0.0, 0.8))]


def measure_workload(model, n_req, lo, hi, new, temperatures, seed=0, layers=0):
    """Continuous batching through ``Engine.run_offline``: N requests with seeded uniform-random prompts of
    MIN..MAX tokens, NEW generated tokens each (no end-of-sequence id, so every request runs its full length),
    wall clock around the whole run; every run is made twice and the second one counts (the first one also captures
    the decode graphs).  One engine serves every temperature; returns one record per temperature."""
    import dataclasses

    import numpy as np
    import torch

    from inf_engine_b200 import Engine, Request, SamplingConfig
    from inf_engine_b200.config import get_preset

    cfg = get_preset(model)
    n_layers_full = cfg.num_hidden_layers
    if layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=layers)
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, n_req)
    n_blocks = int(sum(int(n) + new for n in lens)) // PAGE + 4 * n_req + 64
    torch.cuda.set_device(0)
    engine = Engine.from_random(cfg, seed=seed, dtype="bfloat16", n_total_blocks=n_blocks, block_size=PAGE,
                                max_requests=max(64, n_req), max_tokens_per_step=2048, eos_token=-1)
    out = []
    for temperature in temperatures:
        sampling = SamplingConfig(mode="temperature", temperature=temperature, seed=1) if temperature > 0 else SamplingConfig()

        def once():
            requests = [Request(i, rng.integers(0, cfg.vocab_size, int(n)).tolist(), new, sampling=sampling)
                        for i, n in enumerate(lens)]
            engine.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0}
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = engine.run_offline(requests)
            torch.cuda.synchronize()
            seconds = time.perf_counter() - t0
            engine.completed.clear()
            return seconds, sum(len(v) for v in res.values()), Engine.latency_stats(requests)

        once()
        seconds, generated, lat = once()
        prompt_tokens = int(lens.sum())
        out.append({"seconds": seconds, "generated": generated, "generated_tok_s": generated / seconds,
                    "total_tok_s": (generated + prompt_tokens) / seconds, "prompt_tokens": prompt_tokens,
                    "steps": engine.stats["steps"], "preemptions": engine.stats["preemptions"],
                    "temperature": temperature, "ttft_s_p50": lat["ttft_s"]["p50"], "tpot_s_mean": lat["tpot_s"]["mean"],
                    "layers": cfg.num_hidden_layers, "layers_of_model": n_layers_full})
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    return out


def run_workload(args):
    """``--workload N:MIN:MAX:NEW[:TEMPERATURE]`` with ``--model``: one continuous-batching run (see measure_workload);
    BASELINE.json's other two workloads are ``--model smollm2-1.7b --workload 64:64:2048:256`` and
    ``--model llama-3.2-3b --workload 32:128:4096:128``; the default run prints both under ``workloads``."""
    parts = args.workload.split(":")
    if len(parts) not in (4, 5):
        print("--workload wants N:MIN:MAX:NEW or N:MIN:MAX:NEW:TEMPERATURE")
        return 2
    n_req, lo, hi, new = (int(x) for x in parts[:4])
    temperature = float(parts[4]) if len(parts) == 5 else 0.0
    rec = measure_workload(args.model, n_req, lo, hi, new, (temperature,), args.seed, args.layers)[0]
    print(json.dumps({"impl": "ours", "workload": args.workload, **rec, "dtype": "bf16",
                      "data": "synthetic: seeded random weights, uniform random prompt ids",
                      "config": {"model": args.model, "layers": rec["layers"], "layers_of_model": rec["layers_of_model"],
                                 "requests": n_req, "prompt_min": lo, "prompt_max": hi, "new_tokens": new,
                                 "temperature": temperature, "page_size": PAGE, "max_tokens_per_step": 2048}}))
    return 0


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _reference_package():
    """The reference's ``engine`` package, unmodified, under ``baseline/_ref`` (git-ignored).  It has no setup.py or
    pyproject.toml, so ``pip install --target baseline/_ref`` refuses it; it is pure Python over torch and runs from a
    plain copy of its folder, which is made here when a checkout of the reference lies beside this repository."""
    if not os.path.isfile(os.path.join(REF_DIR, "engine", "llama_paged_engine.py")):
        src = os.environ.get("INF_ENGINE_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
        if not os.path.isfile(os.path.join(src, "engine", "llama_paged_engine.py")):
            return f"no copy of the reference's engine package under baseline/_ref and no checkout at {src}"
        import shutil
        os.makedirs(REF_DIR, exist_ok=True)
        shutil.copytree(os.path.join(src, "engine"), os.path.join(REF_DIR, "engine"))
    return None


def run_reference(args):
    """The reference arm: the UNMODIFIED reference (``baseline/_ref/engine``) through its own public API and stock
    path: ``LlamaModel`` over a ``LlamaWeights`` dictionary of seeded random bfloat16 tensors (built as its own
    tests build one, tests/test_paged_cache.py:42-72) at its ``LLAMA_3_2_1B`` preset (engine/config.py:77-89),
    ``LlamaPagedEngine(model, n_total_blocks, block_size)`` with its defaults (engine/llama_paged_engine.py:129-166),
    prompts through ``submit`` and ``step`` (:169-174, :418-442).  Nothing of this repository's package is imported in
    this process.  Same metric, batch, prompt length, pool and page size as the other arm."""
    why = _reference_package()
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    sys.path.insert(0, REF_DIR)
    try:
        import numpy as np
        import torch
        from engine.config import LLAMA_3_2_1B, LLAMA_3_2_3B, SMOLLM2_1_7B
        from engine.llama_model import LlamaModel
        from engine.llama_paged_engine import LlamaPagedEngine, LlamaRequest
        from engine.llama_weights import LlamaWeights
    except Exception as e:                                   # noqa: BLE001 - whatever keeps it from importing
        print(json.dumps({"impl": "reference", "unavailable": f"the reference does not import here: {e!r}"[:300]}))
        return 0
    presets = {"llama-3.2-1b": LLAMA_3_2_1B, "llama-3.2-3b": LLAMA_3_2_3B, "smollm2-1.7b": SMOLLM2_1_7B}
    if args.model not in presets:
        print(json.dumps({"impl": "reference", "unavailable": f"the reference has no preset for {args.model}"}))
        return 0
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device"}))
        return 0
    cfg = presets[args.model]
    n_layers_full = cfg.n_layer
    if args.layers:
        import dataclasses
        cfg = dataclasses.replace(cfg, n_layer=args.layers)
    pk = peaks()
    dev = "cuda:0"
    torch.cuda.set_device(0)
    g = torch.Generator(device=dev).manual_seed(args.seed)
    d, hq, hk, f, V = cfg.d_model, cfg.n_head * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim, cfg.intermediate_size, cfg.vocab_size

    def mat(*shape):
        return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)

    def gain():
        return (1.0 + (torch.rand(d, generator=g, device=dev) * 0.2 - 0.1)).to(torch.bfloat16)

    tensors = {"model.embed_tokens.weight": mat(V, d), "model.norm.weight": gain()}
    for i in range(cfg.n_layer):
        p = f"model.layers.{i}."
        tensors.update({p + "input_layernorm.weight": gain(), p + "post_attention_layernorm.weight": gain(),
                        p + "self_attn.q_proj.weight": mat(hq, d), p + "self_attn.k_proj.weight": mat(hk, d),
                        p + "self_attn.v_proj.weight": mat(hk, d), p + "self_attn.o_proj.weight": mat(d, hq),
                        p + "mlp.gate_proj.weight": mat(f, d), p + "mlp.up_proj.weight": mat(f, d),
                        p + "mlp.down_proj.weight": mat(d, f)})
    if not cfg.tie_word_embeddings:
        tensors["lm_head.weight"] = mat(V, d)
    model = LlamaModel(LlamaWeights(tensors, cfg), cfg)
    engine = LlamaPagedEngine(model, n_total_blocks=args.pool_requests * POOL_CONTEXT // PAGE, block_size=PAGE)
    rng = np.random.default_rng(args.seed)
    clocks = ClockSampler()
    clocks.start()

    def prompt():
        return rng.integers(0, V, PROMPT_LEN).tolist()

    # prefill: one 2,048-token request that is done after its first token, so step() is its prefill and nothing else
    def prefill_once():
        engine.submit(LlamaRequest(req_id=-1, prompt_ids=prompt(), max_new_tokens=1))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step()
        e1.record()
        torch.cuda.synchronize()
        engine.completed.clear()
        return e0.elapsed_time(e1)

    for _ in range(3):
        prefill_once()
    pre_ms = sorted(prefill_once() for _ in range(args.prefill_reps))
    pre = pre_ms[len(pre_ms) // 2]
    L, H, hd = cfg.n_layer, cfg.n_head, cfg.head_dim
    linear_params = L * ((hq + 2 * hk) * d + d * hq + 3 * f * d)
    flops = 2 * PROMPT_LEN * linear_params + L * 4 * H * hd * (PROMPT_LEN * (PROMPT_LEN + 1) // 2) + 2 * V * d
    prefill = {"value": PROMPT_LEN / pre * 1e3, "unit": "tok/s", "tokens": PROMPT_LEN, "ms": pre,
               "frac": flops / (pre * 1e-3) / (pk["bf16_tflops"] * 1e12), "peak_tflops": pk["bf16_tflops"],
               "peak_source": pk["source"], "note": "flops of the wanted logit row only; the reference computes every row's"}

    def decode(batch, steps, warmup):
        reqs = [LlamaRequest(req_id=i, prompt_ids=prompt(), max_new_tokens=warmup + steps + 8) for i in range(batch)]
        for r in reqs:
            assert engine.submit(r)
        engine.step()                                         # admits and prefills all of them, one decode step
        assert len(engine._active) == batch, "the reference did not admit the whole batch"
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        ctx0 = len(reqs[0].prompt_ids) + len(reqs[0].generated)
        n_before = sum(len(r.generated) for r in reqs)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            engine.step()                                     # reads the sampled ids on the host every step
        e1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        n_tok = sum(len(r.generated) for r in reqs) - n_before
        ms = e0.elapsed_time(e1)
        while engine.has_work:
            engine.step()
        engine.completed.clear()
        return dict(tok_s=n_tok / ms * 1e3, e2e=n_tok / (t1 - t0), ms_per_step=ms / steps, t0=t0, t1=t1,
                    ctx=(ctx0, ctx0 + steps))

    args.warmup = max(args.warmup, 3)
    main = decode(args.batch, args.steps, args.warmup)
    points = {}
    for b in (1, 64):
        if b <= args.pool_requests and not args.no_points:
            # fewer steps: the reference's cache gathers block by block in Python, a second a step at batch 64
            points[f"decode_b{b}"] = decode(b, max(4, args.steps // 16), 3)["tok_s"]
    clocks.stop()
    weight_bytes = 2 * (linear_params + V * d)
    bytes_step = weight_bytes + args.batch * (main["ctx"][0] + args.steps / 2) * (2 * L * hk * 2)
    achieved = bytes_step / (main["ms_per_step"] * 1e-3) / 1e9
    print(json.dumps({
        "metric": "decode tok/s at batch 8 (Llama-3.2-1B size, random weights)", "impl": "reference",
        "value": main["tok_s"], "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights, uniform random prompt ids",
        "config": {"model": args.model, "layers": cfg.n_layer, "layers_of_model": n_layers_full, "hidden": d,
                   "heads": cfg.n_head, "kv_heads": cfg.n_kv_heads, "head_dim": hd, "intermediate": f, "vocab": V,
                   "global_batch": args.batch, "seq_len": PROMPT_LEN, "context_start": main["ctx"][0],
                   "context_end": main["ctx"][1], "pool_context": POOL_CONTEXT, "page_size": PAGE,
                   "parallelism": "single-gpu", "l2": "inputs larger than L2 (weights 2.5 GB per step)",
                   "decode": "the reference's defaults: eager steps, enable_cuda_graphs=False"},
        "e2e": {"value": main["e2e"], "unit": "tok/s", "h2d_bytes_per_step": 8 * args.batch,
                "d2h_bytes_per_step": 8 * args.batch,
                "note": "the reference builds its step tensors from Python lists and reads int64 ids back (.tolist())"},
        "gpu_launches": 0, "launch_note": "library kernels only (torch); none of this repository's",
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "peak_source": pk["source"]},
        "points": points, "clocks": clocks.summary(main["t0"], main["t1"]),
    }))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-3.2-1b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (0: all)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--prefill-reps", type=int, default=7)
    ap.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                    help="measure one part only (short runs for profiling); the JSON line then lacks the rest")
    ap.add_argument("--pool-requests", type=int, default=64, help="requests of 4,096 tokens the cache pool is made for")
    ap.add_argument("--no-points", action="store_true", help="leave out the batch-1 and batch-64 points")
    ap.add_argument("--no-workloads", action="store_true",
                    help="leave out the two continuous-batching workloads at the other models' sizes")
    ap.add_argument("--workload", default=None, metavar="N:MIN:MAX:NEW[:TEMP]",
                    help="instead of the step measurements: N requests through Engine.run_offline (continuous batching)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.workload:
        return run_workload(args)
    args.warmup = max(args.warmup, 3)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
