"""Trace replay: feed given token ids through a model step by step and write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch through the engine's own step function, cache manager and
kernels; nothing is sampled.  For a step that wants logits, `OUT/<step>.f32` holds them as
little-endian 32-bit floats [wanted, vocab] in the order of the entries and of `want`.  After each
step a line `done <step>` is printed and flushed.  `end` lists requests that are finished after the
step; their pages and slot are given back.  The pool holds --max-tokens tokens (each request's
count rounded up to whole pages), so pages are used again.

The reference's nearest tools are `lia forward` / `forward-batch` (src/main.rs:51-133) and its
oracle format of token ids plus `logits.f32` (tests/minicpm5.rs:9-31).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

MAX_LIVE = 4


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time (pool size)")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (divides 64)")
    args = parser.parse_args(argv)
    if args.max_tokens <= 0 or 64 % args.page_size:
        parser.error("--max-tokens must be positive and --page-size must divide 64")

    from .engine import Engine
    from .step import StepEntry

    os.makedirs(args.out, exist_ok=True)
    pool_tokens = (args.max_tokens + 63) // 64 * 64
    engine = Engine(args.model, dtype=args.dtype, page_size=args.page_size, max_tokens=pool_tokens,
                    max_seqs=MAX_LIVE, max_batch_tokens=pool_tokens,
                    max_context=None)
    live = {}                                   # id -> [slot, tokens fed so far]
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            name, tokens = item["id"], [int(t) for t in item["tokens"]]
            if name not in live:
                if len(live) >= MAX_LIVE:
                    raise SystemExit(f"step {step}: more than {MAX_LIVE} live requests")
                live[name] = [engine.admit(), 0]
            slot, fed = live[name]
            if not engine.reserve(slot, fed, fed + len(tokens)):
                raise SystemExit(f"step {step}: the pool of {pool_tokens} tokens has no pages left for request {name}")
            entries.append(StepEntry(slot, tokens, fed, [int(w) for w in item.get("want", [])]))
            live[name][1] = fed + len(tokens)
        logits = engine.step(entries) if entries else None
        if logits is not None and logits.shape[0] > 0:
            data = logits.cpu().numpy().astype("<f4", copy=False)
            data.tofile(os.path.join(args.out, f"{step}.f32"))
        engine.synchronize()
        for name in record.get("end", []):
            if name in live:
                engine.release(live.pop(name)[0])
        sys.stdout.write(f"done {step}\n")
        sys.stdout.flush()
    return 0
