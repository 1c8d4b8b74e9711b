"""Trace replay: feed given token ids through a model step by step and write
logits.  Nothing is sampled.  The program drives the same ``ModelRunner`` —
model, step function, cache and kernels — that generation uses.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch.  For a step that wants something the
float32 logits at the wanted places, in the order of the entries and of
``want``, go to ``<out>/<step>.f32`` as little-endian [wanted, vocab].  After
every step the line ``done <step>`` is printed and flushed.  ``end`` lists
requests whose pages and slot are given back after the step.  The page pool is
made for ``--max-tokens`` tokens (each live request's count rounded up to the
page size), so pages are used again.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

MAX_LIVE_REQUESTS = 64


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (rounded up per request to 64)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    ap.add_argument("--poison-free-pages", action="store_true",
                    help="fill every cache page that no request holds with NaN (at the start and when it is given back)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.page_size <= 0 or 64 % args.page_size:
        ap.error("--page-size must divide 64")

    import torch

    from .. import kernels
    from .batch import StepEntry
    from .runner import ModelRunner

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 2
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    n_pages = max(1, -(-args.max_tokens // args.page_size))
    runner = ModelRunner.from_dir(args.model, dtype=args.dtype, device=args.device, page_size=args.page_size,
                                  n_pages=n_pages, max_requests=MAX_LIVE_REQUESTS,
                                  poison_free_pages=args.poison_free_pages)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if not runner.is_open(rid):
                if not runner.open(rid):
                    raise RuntimeError(f"step {step}: more than {MAX_LIVE_REQUESTS} live requests")
            entries.append(StepEntry(rid, [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        logits = runner.step(entries)
        if logits is not None:
            data = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
            with open(out_dir / f"{step}.f32", "wb") as f:
                f.write(data.tobytes())
        else:
            torch.cuda.synchronize()
        kernels.check_device_errors()
        for rid in rec.get("end", []):
            if runner.is_open(rid):
                runner.close(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
