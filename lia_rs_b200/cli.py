"""`lia`: the command line, in the manner of the reference's (src/main.rs:6-133).

  lia generate MODEL [CONTEXT] --prompt-ids 1,2,3 [--prompt-ids ...] [request and service options]
  lia forward MODEL TOKEN_IDS          top-10 logits at each position, token by token
  lia forward-batch MODEL TOKEN_IDS    argmax at each position of one whole prompt, with seconds
  lia random-model CONFIG_JSON OUT [--seed N]    write a model folder with random weights
  lia inspect MODEL                    the typed configuration and the tensor list

Service options as in `lia serve` (src/server/options.rs:24-76): --max-sequences N (1..64, default
8), --kv-pool-tokens N (default 65536); CONTEXT is positional (default 16384).  Request options carry
the request fields' names: --max-tokens, --temperature, --top-k, --top-p, --seed,
--presence-penalty.  LIA_SAMPLER=mt19937|murmur3_gumbel and LIA_PREFILL_BATCH are read as the
reference reads them.  The reference tokenises text; this engine takes comma-separated token ids.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _ids(text: str) -> list:
    try:
        return [int(t) for t in text.split(",") if t.strip() != ""]
    except ValueError:
        raise SystemExit("expected comma-separated token IDs")


def _prefill_batch() -> int:
    value = os.environ.get("LIA_PREFILL_BATCH")
    if value is None:
        return 512
    batch = int(value)
    if not 128 <= batch <= 4096:
        raise SystemExit("LIA_PREFILL_BATCH must be 128..=4096")
    return batch


def cmd_generate(args) -> int:
    from .engine.generate import Generator
    sampler = os.environ.get("LIA_SAMPLER", "mt19937")
    if sampler not in ("mt19937", "murmur3_gumbel"):
        raise SystemExit(f"invalid LIA_SAMPLER: {sampler}")
    generator = Generator(args.model, dtype=args.dtype, context=args.context, max_sequences=args.max_sequences,
                          kv_pool_tokens=args.kv_pool_tokens, prefill_batch=_prefill_batch(),
                          page_size=args.page_size)
    prompts = [_ids(p) for p in args.prompt_ids]
    started = time.perf_counter()
    outputs = generator.generate(prompts, max_tokens=args.max_tokens, temperature=args.temperature,
                                 top_k=args.top_k, top_p=args.top_p, seed=args.seed,
                                 presence_penalty=args.presence_penalty, sampler=sampler)
    seconds = time.perf_counter() - started
    for i, tokens in enumerate(outputs):
        print(f"request={i} tokens={','.join(str(t) for t in tokens)}")
    count = sum(len(t) for t in outputs)
    print(f"generated={count} seconds={seconds:.6f} preemptions={generator.last_scheduler.stats['preemptions']}",
          file=sys.stderr)
    return 0


def _engine(model, dtype, tokens):
    from .engine import Engine
    pool = (max(len(tokens), 64) + 63) // 64 * 64
    return Engine(model, dtype=dtype, max_tokens=pool, max_seqs=1, max_batch_tokens=pool)


def cmd_forward(args) -> int:
    from .engine import StepEntry
    tokens = _ids(args.token_ids)
    started = time.perf_counter()
    engine = _engine(args.model, args.dtype, tokens)
    print(f"load_seconds={time.perf_counter() - started}", file=sys.stderr)
    slot = engine.admit()
    for position, token in enumerate(tokens):
        started = time.perf_counter()
        engine.reserve(slot, position, position + 1)
        row = engine.logits_to_host(engine.step([StepEntry(slot, [token], position, [0])]))[0]
        print(f"position={position} forward_seconds={time.perf_counter() - started}", file=sys.stderr)
        order = sorted(range(len(row)), key=lambda i: -row[i])[:10]
        print(f"position={position}")
        for i in order:
            print(f"{i} {row[i]}")
    return 0


def cmd_forward_batch(args) -> int:
    from .engine import StepEntry
    tokens = _ids(args.token_ids)
    engine = _engine(args.model, args.dtype, tokens)
    slot = engine.admit()
    engine.reserve(slot, 0, len(tokens))
    started = time.perf_counter()
    rows = engine.logits_to_host(engine.step([StepEntry(slot, tokens, 0, list(range(len(tokens))))]))
    print(f"batch={len(tokens)} seconds={time.perf_counter() - started}", file=sys.stderr)
    for position, row in enumerate(rows):
        best = row.max()
        token = max(i for i in range(len(row)) if row[i] == best)
        print(f"position={position} token={token} logit={row[token]}")
    return 0


def cmd_random_model(args) -> int:
    from .config import resolve_architecture
    from .weights import write_random_model
    with open(args.config, "r", encoding="utf-8") as f:
        raw = json.load(f)
    config = resolve_architecture(raw).config_class.from_dict(raw)
    print(write_random_model(config, args.out, seed=args.seed))
    return 0


def cmd_inspect(args) -> int:
    from .config import read_config_json, resolve_architecture
    raw = read_config_json(args.model)
    arch = resolve_architecture(raw)
    config = arch.config_class.from_dict(raw)
    print(f"architecture={arch.name}")
    for key, value in config.to_dict().items():
        print(f"{key}={value}")
    for spec in arch.build(config).tensor_specs():
        print(f"tensor {spec.name} {list(spec.shape)}")
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="lia", description="lia.rs-style inference on one B200")
    sub = parser.add_subparsers(dest="command", required=True)

    def common(p):
        p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])

    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    g.add_argument("model")
    g.add_argument("context", nargs="?", type=int, default=16384)
    g.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids (repeatable)")
    g.add_argument("--max-tokens", type=int, default=8192)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=42)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--max-sequences", type=int, default=8)
    g.add_argument("--kv-pool-tokens", type=int, default=65536)
    g.add_argument("--page-size", type=int, default=16)
    common(g)
    g.set_defaults(run=cmd_generate)
    for name, fn in (("forward", cmd_forward), ("forward-batch", cmd_forward_batch)):
        p = sub.add_parser(name)
        p.add_argument("model")
        p.add_argument("token_ids")
        common(p)
        p.set_defaults(run=fn)
    r = sub.add_parser("random-model")
    r.add_argument("config")
    r.add_argument("out")
    r.add_argument("--seed", type=int, default=0)
    r.set_defaults(run=cmd_random_model)
    i = sub.add_parser("inspect")
    i.add_argument("model")
    i.set_defaults(run=cmd_inspect)
    args = parser.parse_args(argv)
    return args.run(args)


if __name__ == "__main__":
    sys.exit(main())
