"""Trace replay: feed given token ids through a model step by step and write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--max-live 4] [--page-size 16]

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch through the engine's own step function, cache manager and
kernels; nothing is sampled.  For a step that wants logits, `OUT/<step>.f32` holds them as
little-endian 32-bit floats [wanted, vocab] in the order of the entries and of `want`.  After each
step a line `done <step>` is printed and flushed.  `end` lists requests that are finished after the
step; their pages and slot are given back.  The pool holds --max-tokens tokens, each live request's
count rounded up to a multiple of 64 (or of the page size, if that is larger), so pages are used again.
When the input ends, `OUT/index.json` says which (request, position) each row of each file holds.

`replay(model, steps, ...)` is the same in Python: it returns the rows and the index instead of files.

The reference's nearest tools are `lia forward` / `forward-batch` (src/main.rs:51-133) and its
oracle format of token ids plus `logits.f32` (tests/minicpm5.rs:9-31).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


class TraceError(RuntimeError):
    pass


class TraceRunner:
    """Requests by name over an `Engine`: admits a name at its first entry, reserves pages for every entry,
    runs a step's entries as one batch, releases at `end`.  It has no forward pass, cache or loader of its
    own."""

    def __init__(self, model: str, dtype: str, max_tokens: int, max_live: int = 4, page_size: int = 16, device="cuda:0"):
        from .engine import Engine
        if max_tokens <= 0 or max_live <= 0 or page_size <= 0:
            raise TraceError("max_tokens, max_live and page_size must be positive")
        # `max_tokens` counts every live request rounded up to a multiple of 64 tokens (to whole pages, if a page
        # is larger): the pool gets the whole pages that each such 64 tokens may need
        if page_size >= 64:
            pages = (max_tokens + page_size - 1) // page_size
        else:
            pages = ((max_tokens + 63) // 64) * ((64 + page_size - 1) // page_size)
        self.pool_tokens = pages * page_size
        self.engine = Engine(model, dtype=dtype, device=device, page_size=page_size, max_tokens=self.pool_tokens,
                             max_seqs=max_live, max_batch_tokens=self.pool_tokens, max_context=None)
        self.max_live = max_live
        self.live = {}                               # id -> [slot, tokens fed so far]
        self.index = {}                              # step -> [[id, position], ...] in row order

    def step(self, record: dict):
        """Run one step of the trace; returns its logits [wanted, vocab] (numpy, 32-bit) or None."""
        from .step import StepEntry
        number = record["step"]
        entries, rows = [], []
        for item in record.get("entries", []):
            name, tokens = item["id"], [int(t) for t in item["tokens"]]
            if name not in self.live:
                if len(self.live) >= self.max_live:
                    raise TraceError(f"step {number}: more than {self.max_live} live requests")
                self.live[name] = [self.engine.admit(), 0]
            slot, fed = self.live[name]
            if not self.engine.reserve(slot, fed, fed + len(tokens)):
                raise TraceError(f"step {number}: the pool of {self.pool_tokens} tokens has no pages left for "
                                 f"request {name}")
            want = [int(w) for w in item.get("want", [])]
            entries.append(StepEntry(slot, tokens, fed, want))
            rows += [[name, fed + w] for w in want]
            self.live[name][1] = fed + len(tokens)
        logits = self.engine.step(entries) if entries else None
        data = None
        if logits is not None and logits.shape[0] > 0:
            data = logits.cpu().numpy().astype("<f4", copy=True)
            self.index[str(number)] = rows
        self.engine.synchronize()
        for name in record.get("end", []):
            if name in self.live:
                self.engine.release(self.live.pop(name)[0])
        return data


def replay(model: str, steps, dtype: str = "bfloat16", max_tokens: int = 4096, max_live: int = 4, page_size: int = 16):
    """Replay `steps` (dicts of the form above) through the model folder `model`.  Returns
    (logits, index): `logits[step]` is the step's array [wanted, vocab], `index[step]` lists the
    (request, position) of each of its rows."""
    runner = TraceRunner(model, dtype, max_tokens, max_live, page_size)
    logits = {}
    for record in steps:
        data = runner.step(record)
        if data is not None:
            logits[record["step"]] = data
    return logits, {int(k) if k.lstrip("-").isdigit() else k: v for k, v in runner.index.items()}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files and index.json")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time (pool size)")
    parser.add_argument("--max-live", type=int, default=4, help="most requests live at a time (request slots)")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    args = parser.parse_args(argv)
    if args.max_tokens <= 0 or args.max_live <= 0 or args.page_size <= 0:
        parser.error("--max-tokens, --max-live and --page-size must be positive")
    os.makedirs(args.out, exist_ok=True)
    try:
        runner = TraceRunner(args.model, args.dtype, args.max_tokens, args.max_live, args.page_size)
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            data = runner.step(record)
            if data is not None:
                data.tofile(os.path.join(args.out, f"{record['step']}.f32"))
            sys.stdout.write(f"done {record['step']}\n")
            sys.stdout.flush()
    except TraceError as error:
        raise SystemExit(str(error))
    with open(os.path.join(args.out, "index.json"), "w", encoding="utf-8") as f:
        json.dump({"vocab_size": runner.engine.spec.vocab_size, "dtype": "float32", "rows": runner.index}, f)
    return 0
