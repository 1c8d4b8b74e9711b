"""Command line: generate from a model folder or from a preset with random weights.

Options follow the reference's entry points where it has them:
``--model``, ``--prompt``, ``--n``, ``--mode``, ``--top-p``, ``--top-k``, ``--seed``
(scripts/generate_llama.py:26-34); ``--model-dir``, ``--max-new-tokens``,
``--max-ctx``, ``--device``, ``--repetition-penalty`` (main.py:498-582);
``--n-total-blocks``, ``--block-size`` (server.py:100-105).  The reference has no
temperature flag and no way to give token ids; ``--temperature``,
``--prompt-ids`` and the engine options are added here.

    bin/generate_llama --model tiny-a --random-weights --prompt-ids 5,17,3 --n 8
    bin/generate_llama --model-dir DIR --prompt "The capital of France is" --mode top_p --top-p 0.9
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="generate_llama", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", default=None, help="preset name (see --list-presets) or a model folder")
    p.add_argument("--model-dir", default=None, help="folder with config.json and safetensors")
    p.add_argument("--random-weights", action="store_true", help="seeded random weights for --model preset")
    p.add_argument("--weights-seed", type=int, default=0)
    p.add_argument("--prompt", default=None, help="text; needs tokenizer files in the model folder")
    p.add_argument("--prompt-ids", default=None, help="comma-separated token ids; ';' separates several prompts")
    p.add_argument("--prompt-file", default=None, help="file with one prompt of comma-separated ids per line")
    p.add_argument("--n", "--max-new-tokens", dest="n", type=int, default=50, help="new tokens to generate")
    p.add_argument("--mode", choices=["greedy", "temperature", "top_k", "top_p"], default="greedy")
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--top-k", type=int, default=50)
    p.add_argument("--repetition-penalty", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=0, help="sampling seed")
    p.add_argument("--dtype", choices=["bfloat16", "float32", "bf16", "fp32"], default="bfloat16")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--max-ctx", type=int, default=None, help="size the cache pool for this many tokens")
    p.add_argument("--n-total-blocks", type=int, default=None, help="pages in the cache pool")
    p.add_argument("--block-size", type=int, default=16, help="tokens per page")
    p.add_argument("--max-batch", type=int, default=64)
    p.add_argument("--max-tokens-per-step", type=int, default=2048)
    p.add_argument("--chunk", type=int, default=None, help="largest prompt portion of one request in a step")
    p.add_argument("--eos-id", type=int, default=None)
    p.add_argument("--stats-json", default=None, help="write timing and engine counters here")
    p.add_argument("--trace-jsonl", default=None, help="write one JSON line per engine step here (batch make-up, pages free, host time)")
    p.add_argument("--nvtx", action="store_true", help="an NVTX range around every engine step, for a timeline tool")
    p.add_argument("--checks", action="store_true",
                   help="a checks build of the kernels: every page id, cache slot and token id they read is compared with "
                        "the pool and the vocabulary; one out of range is reported and not used (slower; for debugging)")
    p.add_argument("--list-presets", action="store_true")
    return p


def _parse_ids(text: str) -> list[list[int]]:
    return [[int(t) for t in part.replace(" ", "").split(",") if t] for part in text.split(";") if part.strip()]


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from ..config.registry import get_preset, preset_names
    from ..engine.engine import Engine
    from ..engine.scheduler import Request
    from ..sampling.sampler import SamplingConfig

    if args.list_presets:
        print("\n".join(preset_names()))
        return 0
    model_dir = args.model_dir or (args.model if args.model and Path(args.model).is_dir() else None)
    prompts: list[list[int]] = []
    tokenizer = None
    if args.prompt_ids:
        prompts = _parse_ids(args.prompt_ids)
    elif args.prompt_file:
        prompts = _parse_ids(";".join(Path(args.prompt_file).read_text().splitlines()))
    elif args.prompt is not None:
        if model_dir is None or not any((Path(model_dir) / f).is_file() for f in ("tokenizer.json", "tokenizer.model")):
            print("--prompt needs tokenizer files in the model folder; give --prompt-ids instead", file=sys.stderr)
            return 2
        from transformers import AutoTokenizer   # tokenising only, as scripts/generate_llama.py:56-59

        tokenizer = AutoTokenizer.from_pretrained(str(model_dir))
        prompts = [tokenizer.encode(args.prompt)]
    else:
        print("give --prompt-ids, --prompt-file or --prompt", file=sys.stderr)
        return 2

    longest = max(len(p) for p in prompts) + args.n + 1
    if args.n_total_blocks is not None:
        n_blocks = args.n_total_blocks
    else:
        per = args.max_ctx or longest
        n_blocks = -(-per // args.block_size) * min(len(prompts), args.max_batch)
    kw = dict(dtype=args.dtype, device=args.device, n_total_blocks=n_blocks, block_size=args.block_size,
              max_requests=args.max_batch, eos_token=args.eos_id, max_tokens_per_step=args.max_tokens_per_step,
              chunk=args.chunk, trace_path=args.trace_jsonl, nvtx=args.nvtx)
    if args.checks:
        from .. import kernels
        kernels.enable_checks()
    t0 = time.perf_counter()
    if model_dir is not None:
        engine = Engine.from_dir(model_dir, **kw)
    elif args.model and args.random_weights:
        engine = Engine.from_random(get_preset(args.model), seed=args.weights_seed, **kw)
    else:
        print("give --model-dir DIR, or --model PRESET --random-weights", file=sys.stderr)
        return 2
    t_load = time.perf_counter() - t0
    sampling = SamplingConfig(mode=args.mode, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                              repetition_penalty=args.repetition_penalty, seed=args.seed)
    requests = [Request(req_id=i, prompt_ids=p, max_new_tokens=args.n, sampling=sampling) for i, p in enumerate(prompts)]
    t0 = time.perf_counter()
    out = engine.run_offline(requests)
    t_gen = time.perf_counter() - t0
    for r in requests:
        if r.error:
            print(f"request {r.req_id}: refused: {r.error}", file=sys.stderr)
            continue
        ids = out[r.req_id]
        if tokenizer is not None:
            print("Output:", tokenizer.decode(ids))
        print(f"{r.req_id}: " + ",".join(str(t) for t in ids))
    n_new = sum(len(v) for v in out.values())
    print(f"[{n_new} tokens in {t_gen:.3f} s = {n_new / max(t_gen, 1e-9):.1f} tok/s; load {t_load:.2f} s]", file=sys.stderr)
    if args.stats_json:
        Path(args.stats_json).write_text(json.dumps({"load_s": t_load, "generate_s": t_gen, "new_tokens": n_new,
                                                     **engine.stats, **engine.latency_stats(requests)}, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
