#!/usr/bin/env python3
"""Decode and prefill throughput of the 2B-class MiniCPM5 Llama configuration on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

A "step" is one decode step of `--batch` requests, each with a 2,048-token uniform-random prompt in
the cache (the pool is sized for the 32,768-token context of the configuration).  One JSON line is
printed:

  value      decoded tokens a second, K steps timed on the device with CUDA events (the tokens fed
             are fixed beforehand, so the device never waits for the host)
  e2e        the same through the scheduler that `generate()` runs: every step copies that step's
             token ids, positions and slots from pinned host memory to the device and reads the
             sampled token ids back to the host, which feed the next step
  prefill    one step of a single 2,048-token prompt: tokens/s, ms, and flops / time / peak
  roofline   the decode step's bytes (every weight once + the live requests' cache) / time / peak
  points     decode tokens/s at batch 1 and 64
  kernels    for the decode step and the prefill step, each kernel class's share of the step's device time
             (CUDA events around every launch of a step run launch by launch, `Engine(profile=True)`) and the
             fraction of its own roofline: weight or cache bytes / time / HBM peak for the decode step,
             flops / time / bf16 peak for the prefill step
  checked    outside the timed region, the benchmarked engine runs a 64-token prompt whole and again as 48
             tokens and 16 single tokens; both are compared with the true 32-bit path over the same weights;
             and the timed prompt's logits from the replayed graph are compared with those of its first step,
             which was launched kernel by kernel (`prefill_replayed_vs_launched`)

Every point is timed for at least half a second of device time: the loop of K steps is repeated and the
median loop is reported (`repeats` says how many).  Weights (4.1 GB) and cache are far larger than the
126 MB L2, so no L2 flush is needed between timed steps.  Peaks come from MEASURED_PEAKS.json beside this
file when it exists.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the 2B-class configuration the headline numbers are quoted on
CONFIG_2B = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=2048, intermediate_size=6144,
                 num_hidden_layers=40, num_attention_heads=16, num_key_value_heads=2, head_dim=128,
                 vocab_size=73448, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
                 scale_emb=12, scale_depth=1.4, dim_model_base=256, max_position_embeddings=32768,
                 initializer_range=0.02, hidden_act="silu", torch_dtype="bfloat16")
PROMPT = 2048
PAGE = 16


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], tflops=p["bf16_tflops"], sustained=p.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm=6650.0, tflops=1590.0, sustained=1400.0, source="fallback")


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", "0", "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                         text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        # the clocks of an idle GPU say nothing about the timed kernels: only samples taken under load count
        # (utilisation of at least half; the host-side phases of the run between the timed loops are idle)
        sm, top, reasons, every = [], None, set(), 0
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 10:
                continue
            try:
                clock, top, busy = float(f[1]), float(f[2]), float(f[9])
            except ValueError:
                continue
            every += 1
            if busy < 50.0:
                continue
            sm.append(clock)
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": top, "reasons": sorted(reasons),
                "samples": len(sm), "samples_idle": every - len(sm)}


def model_bytes(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * d * h + nq * d * h + 3 * i * h + 2 * h
    head = v * h                                     # tied: the table is read once, as the output matrix
    return 2 * (layers * per_layer + head + h), 2 * layers * 2 * nkv * d      # weight bytes, cache bytes per token


def prefill_flops(cfg, layers, tokens):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2 * tokens * layers * ((nq + 2 * nkv) * d * h + nq * d * h + 3 * i * h) + 2 * v * h
    attention = layers * 4 * nq * d * tokens * (tokens + 1) / 2
    return linear + attention


def fill(engine, batch, prompt_tokens, rng_seed):
    """Admit `batch` requests and put their prompts' keys and values in the cache by real prefill."""
    import numpy as np
    from lia_rs_b200.engine import StepEntry
    rng = np.random.default_rng(rng_seed)
    slots = []
    vocab = engine.spec.vocab_size
    for _ in range(batch):
        slot = engine.admit()
        tokens = [int(t) for t in rng.integers(0, vocab, size=prompt_tokens)]
        assert engine.reserve(slot, 0, prompt_tokens)
        engine.step([StepEntry(slot, tokens, 0, [])])
        slots.append(slot)
    engine.synchronize()
    return slots


MIN_TIMED_MS = 500.0          # device time every point is measured over, at least
MAX_DECODE_STEPS = 512        # steps a point may take in all (its requests' pages are reserved for them)


def time_decode(engine, slots, start, steps, warmup):
    """Device time per step of the median loop of `steps` decode steps, after `warmup` untimed steps; the loop is
    repeated until MIN_TIMED_MS of device time have been measured (within MAX_DECODE_STEPS).  Tokens are fixed
    beforehand.  Returns (ms per step, kernels per step, repeats, steps run in all)."""
    import numpy as np
    import torch
    from lia_rs_b200.engine import StepEntry
    from lia_rs_b200.kernels import ops
    rng = np.random.default_rng(1)
    vocab = engine.spec.vocab_size
    most = max(warmup + steps, MAX_DECODE_STEPS)
    feed = rng.integers(0, vocab, size=(most, len(slots)))
    for slot in slots:
        assert engine.reserve(slot, start, start + most)
    picked = torch.empty(len(slots), dtype=torch.int32, device=engine.device)
    done = 0

    def run(count):
        nonlocal done
        for _ in range(count):
            entries = [StepEntry(slot, [int(feed[done, j])], start + done, [0]) for j, slot in enumerate(slots)]
            logits = engine.step(entries)
            ops.select_tokens(logits, picked)
            done += 1

    run(warmup)
    loops, launches, measured = [], 0, 0.0
    while True:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        before = engine.stats["kernels"]
        begin.record()
        run(steps)
        end.record()
        torch.cuda.synchronize()
        engine.synchronize()
        loops.append(begin.elapsed_time(end))
        measured += loops[-1]
        # kernels of the model's step (counted at the launch sites; a graph replay adds its kernel nodes) + selection
        launches = (engine.stats["kernels"] - before) // steps + 1
        if measured >= MIN_TIMED_MS or done + steps > most:
            break
    return statistics.median(loops) / steps, launches, len(loops), done


def time_e2e(engine, batch, steps, warmup):
    """Wall time per decode step through the scheduler: host token ids in, host token ids out.  The loop of
    `steps` steps is repeated as `time_decode` repeats its loop; the median loop is reported."""
    import numpy as np
    import torch
    from lia_rs_b200.engine.scheduler import Scheduler
    rng = np.random.default_rng(2)
    vocab = engine.spec.vocab_size
    scheduler = Scheduler(engine, max_batch_tokens=engine.max_batch_tokens)
    most = max(warmup + steps, MAX_DECODE_STEPS)
    for i in range(batch):
        scheduler.add(i, [int(t) for t in rng.integers(0, vocab, size=PROMPT)], max_tokens=most + batch + 4)
    while any(not r.generated for r in scheduler.live()) or scheduler.queue:
        scheduler.step()
    for _ in range(warmup):
        scheduler.step()
    loops, done, measured = [], warmup, 0.0
    h2d = d2h = 0
    while True:
        torch.cuda.synchronize()
        h2d = d2h = 0
        started = time.perf_counter()
        for _ in range(steps):
            scheduler.step()
            h2d += engine.runtime_step.h2d_bytes
            d2h += 4 * batch
        torch.cuda.synchronize()
        loops.append(time.perf_counter() - started)
        measured += loops[-1] * 1e3
        done += steps
        if measured >= MIN_TIMED_MS or done + steps > most:
            break
    for request in scheduler.live():
        engine.release(request.slot)
    return statistics.median(loops) / steps, h2d // steps, d2h // steps


def time_prefill(engine, warmup=3, repeats=25):
    import numpy as np
    import torch
    from lia_rs_b200.engine import StepEntry
    rng = np.random.default_rng(3)
    tokens = [int(t) for t in rng.integers(0, engine.spec.vocab_size, size=PROMPT)]
    times = []
    k = -1
    first = last = None
    while k + 1 < warmup + repeats or sum(times) < MIN_TIMED_MS:
        k += 1
        slot = engine.admit()
        assert engine.reserve(slot, 0, PROMPT)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        logits = engine.step([StepEntry(slot, tokens, 0, [PROMPT - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.synchronize()
        engine.release(slot)
        if k == 0:
            first = logits.clone()               # launched kernel by kernel: a shape's first step
        last = logits
        if k >= warmup:
            times.append(begin.elapsed_time(end))
    # the same prompt through the replayed graph must give what the step launched kernel by kernel gave (kernels that
    # start under their predecessors' tails must not read what is not written yet)
    drift = float((last.float() - first.float()).abs().max())
    return statistics.median(times), drift


# The family's other sizes and the workloads they are quoted on (--workload): not the contract's line, one line each.
CONFIG_8B = dict(CONFIG_2B, hidden_size=4096, num_attention_heads=32, intermediate_size=16384, num_hidden_layers=32,
                 tie_word_embeddings=False)
CONFIG_05B = dict(CONFIG_2B, hidden_size=1024, num_attention_heads=16, head_dim=64, intermediate_size=4096,
                  num_hidden_layers=24)


def fill_in_portions(engine, batch, prompt_tokens, portion, rng_seed):
    """As `fill`, with prompts longer than a step takes: `portion` tokens a step."""
    import numpy as np
    from lia_rs_b200.engine import StepEntry
    rng = np.random.default_rng(rng_seed)
    slots = []
    for _ in range(batch):
        slot = engine.admit()
        assert engine.reserve(slot, 0, prompt_tokens)
        for start in range(0, prompt_tokens, portion):
            count = min(portion, prompt_tokens - start)
            tokens = [int(t) for t in rng.integers(0, engine.spec.vocab_size, size=count)]
            engine.step([StepEntry(slot, tokens, start, [])])
        slots.append(slot)
    engine.synchronize()
    return slots


def device_trace(run) -> dict:
    """`run()` under a trace of the device's activity (CUPTI through torch's profiler): how long the device was
    busy, and each kernel's share.  Kernels chained with programmatic launch overlap (a successor waits on the device
    for its predecessor), so at every moment the time goes to the kernel that began first among those running; the
    sum of the kernels' own durations would count the waiting twice."""
    import heapq
    import torch
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run()
    spans = sorted((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                   if e.device_type == torch.autograd.DeviceType.CUDA)
    if not spans:
        return {"unavailable": "the profiler recorded no device activity"}
    points = sorted({t for begin, end, _ in spans for t in (begin, end)})
    busy, share, running, k = 0.0, {}, [], 0
    for t0, t1 in zip(points, points[1:]):
        while k < len(spans) and spans[k][0] <= t0:
            heapq.heappush(running, spans[k])
            k += 1
        while running and running[0][1] <= t0:
            heapq.heappop(running)
        if running:
            busy += t1 - t0
            name = running[0][2].replace("void ", "").replace("(anonymous namespace)::", "").split("(")[0]
            share[name] = share.get(name, 0.0) + (t1 - t0)
    span = spans[-1][1] - spans[0][0]
    top = sorted(share.items(), key=lambda item: -item[1])[:12]
    return {"span_s": round(span / 1e6, 3), "busy_s": round(busy / 1e6, 3),
            "kernels_ms": {name: round(t / 1e3, 1) for name, t in top}}


def other_workload(name, steps, warmup, trace=False) -> int:
    import numpy as np
    import torch
    from lia_rs_b200 import LlamaConfig
    from lia_rs_b200.engine import Engine, StepEntry
    from lia_rs_b200.engine.scheduler import Scheduler
    peak = peaks()
    if name in ("8b-decode", "8b-prefill"):
        cfg, batch, prompt = CONFIG_8B, 64, 8192
        layers = cfg["num_hidden_layers"]
        if name == "8b-decode":
            pool = batch * (prompt + MAX_DECODE_STEPS + 64)
            engine = Engine.random(LlamaConfig.from_dict(cfg), seed=5, dtype="bfloat16", page_size=PAGE, max_tokens=pool,
                                   max_seqs=batch, max_batch_tokens=PROMPT, max_context=cfg["max_position_embeddings"])
            slots = fill_in_portions(engine, batch, prompt, PROMPT, 7)
            ms, launches, _, ran = time_decode(engine, slots, prompt, steps, warmup)
            weight_bytes, cache_bytes_per_token = model_bytes(cfg, layers)       # (untied: of the table only a few rows are read)
            step_bytes = weight_bytes + batch * (prompt + (warmup + ran) // 2) * cache_bytes_per_token
            achieved = step_bytes / (ms * 1e-3) / 1e9
            print(json.dumps({"workload": name, "metric": "decode tokens/s (8B-class, batch 64, 8,192-token prompts, bf16)",
                              "value": round(batch * 1000.0 / ms, 1), "ms_per_step": round(ms, 3), "steps": steps,
                              "gpu_launches": int(launches),
                              "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm"], "unit": "GB/s",
                                           "frac": round(achieved / peak["hbm"], 4)}}))
            return 0
        context = cfg["max_position_embeddings"]
        engine = Engine.random(LlamaConfig.from_dict(cfg), seed=5, dtype="bfloat16", page_size=PAGE, max_tokens=context,
                               max_seqs=1, max_batch_tokens=PROMPT, max_context=context)
        rng = np.random.default_rng(3)
        times = []
        for repeat in range(2):
            slot = engine.admit()
            assert engine.reserve(slot, 0, context)
            times = []
            for start in range(0, context, PROMPT):
                tokens = [int(t) for t in rng.integers(0, cfg["vocab_size"], size=PROMPT)]
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                begin.record()
                engine.step([StepEntry(slot, tokens, start, [PROMPT - 1] if start + PROMPT == context else [])])
                end.record()
                torch.cuda.synchronize()
                times.append(begin.elapsed_time(end))
            engine.synchronize()
            engine.release(slot)
        linear = prefill_flops(cfg, layers, PROMPT) - layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * PROMPT * (PROMPT + 1) / 2
        print(json.dumps({"workload": name, "metric": "prefill in 2,048-token portions up to 32,768 tokens (8B-class, bf16)",
                          "value": round(context * 1000.0 / sum(times), 1), "unit": "tokens/s",
                          "ms_first_portion": round(times[0], 2), "ms_last_portion": round(times[-1], 2),
                          "frac_first_portion": round(prefill_flops(cfg, layers, PROMPT) / (times[0] * 1e-3) / (peak["tflops"] * 1e12), 4),
                          "linear_tflop_per_portion": round(linear / 1e12, 2)}))
        return 0
    if name == "0.5b-mixed":
        cfg, requests, decode_tokens = CONFIG_05B, 64, 256
        rng = np.random.default_rng(4)
        prompts = [[int(t) for t in rng.integers(0, cfg["vocab_size"], size=int(rng.integers(16, 4097)))] for _ in range(requests)]
        pool = 160 * 1024
        engine = Engine.random(LlamaConfig.from_dict(cfg), seed=4, dtype="bfloat16", page_size=PAGE, max_tokens=pool,
                               max_seqs=requests, max_batch_tokens=PROMPT, max_context=cfg["max_position_embeddings"])
        result = {}
        for repeat in range(3 if trace else 2):      # the first pass compiles nothing but allocates and captures
            scheduler = Scheduler(engine, max_batch_tokens=PROMPT)
            for i, prompt in enumerate(prompts):
                scheduler.add(i, prompt, max_tokens=decode_tokens)
            torch.cuda.synchronize()
            if trace and repeat == 2:                # a third pass under the trace; the line's figures are the second's
                result["device_trace"] = device_trace(lambda: (scheduler.run(), torch.cuda.synchronize()))
                break
            started = time.perf_counter()
            scheduler.run()
            torch.cuda.synchronize()
            seconds = time.perf_counter() - started
            generated = sum(len(r.generated) for r in scheduler.finished)
            result = {"workload": name,
                      "metric": "generated tokens/s through the scheduler (0.5B-class, 64 requests, prompts U[16, 4096], 256 tokens each, bf16)",
                      "value": round(generated / seconds, 1), "unit": "tokens/s", "seconds": round(seconds, 3),
                      "prompt_tokens": sum(len(p) for p in prompts), "generated_tokens": generated,
                      "steps": scheduler.stats["steps"], "pipelined_steps": scheduler.stats["pipelined_steps"],
                      "preemptions": scheduler.stats["preemptions"], "kv_pool_tokens": pool}
        print(json.dumps(result))
        return 0
    print(f"bench.py: unknown workload {name!r}")
    return 2


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=CONFIG_2B["num_hidden_layers"],
                        help="run fewer layers than the configuration's 40 (both numbers are reported)")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-points", action="store_true", help="skip batch 1 and batch 64")
    parser.add_argument("--workload", default=None, choices=["8b-decode", "8b-prefill", "0.5b-mixed"],
                        help="one of the family's other sizes on the workload it is quoted on (prints its own line)")
    parser.add_argument("--device-trace", action="store_true",
                        help="with --workload 0.5b-mixed: one more pass under a trace of the device's kernels; adds "
                             "the device's busy time and each kernel's share of it to the line")
    parser.add_argument("--no-check", action="store_true", help="skip the comparison with the 32-bit path")
    parser.add_argument("--no-graphs", action="store_true",
                        help="launch decode steps kernel by kernel instead of replaying CUDA graphs (for profilers)")
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "Heltion/lia.rs is a Rust crate (nightly toolchain + NVIDIA cuda-rust git dependency, no "
                          "Python package); pip cannot install it offline and no cargo/rustc exists in this image"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.workload:
        return other_workload(args.workload, args.steps, args.warmup, trace=args.device_trace)

    import torch
    from lia_rs_b200 import LlamaConfig
    from lia_rs_b200.engine import Engine
    from lia_rs_b200.weights import random_weights

    cfg = dict(CONFIG_2B, num_hidden_layers=args.layers)
    config = LlamaConfig.from_dict(cfg)
    peak = peaks()
    sampler = ClockSampler()
    sampler.start()                                  # clocks over the whole run
    largest = args.batch if args.no_points else max(args.batch, 64)
    most_steps = max(args.steps + args.warmup, MAX_DECODE_STEPS)
    pool = largest * ((PROMPT + most_steps + 8 + 63) // 64 * 64) + PROMPT
    tensors = random_weights(config, seed=0)         # one set of weights for the benchmarked engine and for its check
    engine = Engine.from_tensors(config, tensors, dtype="bfloat16", page_size=PAGE, max_tokens=pool, max_seqs=largest,
                                 max_batch_tokens=PROMPT, max_context=cfg["max_position_embeddings"],
                                 cuda_graphs=not args.no_graphs)
    weight_bytes, cache_bytes_per_token = model_bytes(cfg, args.layers)

    def decode_point(batch, steps, warmup):
        slots = fill(engine, batch, PROMPT, 10 + batch)
        result = time_decode(engine, slots, PROMPT, steps, warmup)
        for slot in slots:
            engine.release(slot)
        return result

    ms, launches, repeats, ran = decode_point(args.batch, args.steps, args.warmup)
    value = args.batch * 1000.0 / ms
    context = PROMPT + (args.warmup + ran) // 2
    step_bytes = weight_bytes + args.batch * context * cache_bytes_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    e2e_s, h2d, d2h = time_e2e(engine, args.batch, args.steps, args.warmup)
    prefill_ms, prefill_drift = time_prefill(engine)
    flops = prefill_flops(cfg, args.layers, PROMPT)
    points = {}
    if not args.no_points:
        for batch in (1, 64):
            point_ms, _, _, _ = decode_point(batch, args.steps, args.warmup)
            points[f"decode_b{batch}"] = round(batch * 1000.0 / point_ms, 1)
    kernels = kernel_shares(engine, args.batch, peak)
    checked = None if args.no_check else check_against_32_bit(engine, config, tensors, cfg)
    if checked is not None:
        checked["prefill_replayed_vs_launched"] = prefill_drift
        checked["ok"] = bool(checked["ok"] and prefill_drift <= 1e-3)
    clocks = sampler.stop()

    line = {
        "metric": "decode tokens/s (2B-class MiniCPM5 Llama, batch %d, 2,048-token prompts, bf16, one B200)" % args.batch,
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "repeats": repeats, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random-init weights N(0, 0.02)",
        "impl": "ours",
        "config": {"model": "MiniCPM5-Llama-2B-class", "layers": args.layers, "layers_of_config": 40,
                   "hidden": 2048, "heads": 16, "kv_heads": 2, "head_dim": 128, "intermediate": 6144,
                   "vocab": 73448, "tied_head": True, "global_batch": args.batch, "seq_len": PROMPT,
                   "context_length": cfg["max_position_embeddings"], "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (4.1 GB weights + cache per step)", "peaks": peak["source"]},
        "e2e": {"value": round(args.batch / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "prefill": {"value": round(PROMPT * 1000.0 / prefill_ms, 1), "tokens": PROMPT, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["tflops"] * 1e12), 4),
                    # the same against the library product's rate in a seconds-long loop under the power cap
                    "frac_of_sustained": (round(flops / (prefill_ms * 1e-3) / (peak["sustained"] * 1e12), 4)
                                          if peak.get("sustained") else None)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm"], 4)},
        "points": points,
        "kernels": kernels,
        "checked": checked,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


def kernel_shares(engine, batch, peak):
    """Per kernel class, for a decode step of `batch` requests and for the 2,048-token prefill step: its share of
    the step's device time and the fraction of its own roofline.  The steps run launch by launch with CUDA
    events around every launch (`engine.profile`), outside every timed region."""
    import numpy as np
    from lia_rs_b200.engine import StepEntry
    rng = np.random.default_rng(5)
    vocab = engine.spec.vocab_size
    slots = fill(engine, batch, PROMPT, 30)
    for slot in slots:
        assert engine.reserve(slot, PROMPT, PROMPT + 8)
    engine.profile = True
    out = {}
    try:
        for k in range(8):
            engine.step([StepEntry(slot, [int(rng.integers(0, vocab))], PROMPT + k, [0]) for slot in slots])
            if k == 2:
                engine.profile_summary()                  # the first steps allocate: not counted
        summary = engine.profile_summary()
        total = sum(v["ms"] for v in summary.values())
        out["decode"] = {name: {"share": round(v["ms"] / total, 4),
                                "frac": round(v["bytes"] / (v["ms"] * 1e-3) / 1e9 / peak["hbm"], 4) if v["bytes"] else None}
                         for name, v in sorted(summary.items())}
        for slot in slots:
            engine.release(slot)
        tokens = [int(t) for t in rng.integers(0, vocab, size=PROMPT)]
        for k in range(3):
            slot = engine.admit()
            assert engine.reserve(slot, 0, PROMPT)
            engine.step([StepEntry(slot, tokens, 0, [PROMPT - 1])])
            engine.synchronize()
            engine.release(slot)
            if k == 0:
                engine.profile_summary()
        summary = engine.profile_summary()
        total = sum(v["ms"] for v in summary.values())
        out["prefill"] = {name: {"share": round(v["ms"] / total, 4),
                                 "frac": round(v["flops"] / (v["ms"] * 1e-3) / 1e12 / peak["tflops"], 4) if v["flops"] else None}
                          for name, v in sorted(summary.items())}
    finally:
        engine.profile = False
    return out


def check_against_32_bit(engine, config, tensors, cfg):
    """A tripwire, not parity (the tests hold that): the benchmarked bfloat16 engine and the true 32-bit path over
    the same weights, a 64-token prompt whole and again as 48 tokens and 16 single tokens.  The limit is what 16-bit
    rounding at six places a layer adds up to over the layers, at the size of the largest logit."""
    import math
    import numpy as np
    import torch
    from lia_rs_b200.engine import Engine, StepEntry
    rng = np.random.default_rng(6)
    tokens = [int(t) for t in rng.integers(0, cfg["vocab_size"], size=64)]

    def both_ways(e):
        slot = e.admit()
        assert e.reserve(slot, 0, 64)
        whole = e.step([StepEntry(slot, tokens, 0, list(range(64)))]).float().cpu()
        e.synchronize()
        e.release(slot)
        slot = e.admit()
        assert e.reserve(slot, 0, 64)
        rows = [e.step([StepEntry(slot, tokens[:48], 0, list(range(48)))]).float().cpu()]
        for i in range(48, 64):
            rows.append(e.step([StepEntry(slot, [tokens[i]], i, [0])]).float().cpu())
        e.synchronize()
        e.release(slot)
        return whole, torch.cat(rows)

    whole, cut = both_ways(engine)
    exact_engine = Engine.from_tensors(config, tensors, dtype="float32", page_size=PAGE, max_tokens=128, max_seqs=2,
                                       max_batch_tokens=64, max_context=cfg["max_position_embeddings"])
    exact, exact_cut = both_ways(exact_engine)
    del exact_engine
    torch.cuda.empty_cache()
    largest = float(exact.abs().max())
    limit = 2.0 ** -8 * math.sqrt(6 * cfg["num_hidden_layers"]) * largest
    worst = max(float((whole - exact).abs().max()), float((cut - exact).abs().max()))
    return {"max_abs_err": round(worst, 5), "limit": round(limit, 5), "largest_logit": round(largest, 4),
            "whole_vs_cut_32_bit": float((exact - exact_cut).abs().max()), "ok": bool(worst <= limit)}


if __name__ == "__main__":
    sys.exit(main())
