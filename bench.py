#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-0.5B sizes with random
weights on one B200.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A "step" is one decode step of the whole batch.  `value` is decoded tokens a
second timed on the device over K steps that never return to the host
(`Engine.decode_steps`); `e2e` is the same through the scheduler that the Python
entry point (`generate_batch`) runs: prompts come from the host, every step's
positions, slots and block tables are copied from pinned host memory and its
sampled ids are read back by the host, which judges the ends one step behind.  The line also carries the prefill of 2,048 tokens, the decode
roofline and decode at batch 1 and 64.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Qwen2.5-0.5B sizes
SIZES = dict(num_hidden_layers=24, hidden_size=896, num_attention_heads=14, num_key_value_heads=2,
             head_dim=64, intermediate_size=4864, vocab_size=151936, rope_theta=1000000.0,
             rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=32768,
             use_sliding_window=False, sliding_window=32768, max_window_layers=24)
PROMPT_LEN, NEW_TOKENS, PREFILL_TOKENS, PAGE = 512, 256, 2048, 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            raw = json.load(open(path))
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in raw.items() if k in out and v})
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def weight_bytes(cfg, layers):
    """Bytes of weights one decode step reads: every matrix once (bfloat16),
    gains and biases in float32."""
    h, d = cfg["hidden_size"], cfg["head_dim"]
    q, kv, inner = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d, cfg["intermediate_size"]
    per_layer = 2 * ((q + 2 * kv) * h + h * q + 3 * inner * h) + 4 * ((q + 2 * kv) + 2 * h)
    head = 2 * cfg["vocab_size"] * h
    return layers * per_layer + head + 4 * h


def kv_bytes_per_token(cfg, layers):
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, layers, tokens):
    h, d = cfg["hidden_size"], cfg["head_dim"]
    q, kv, inner = cfg["num_attention_heads"] * d, cfg["num_key_value_heads"] * d, cfg["intermediate_size"]
    linear = 2 * tokens * ((q + 2 * kv) * h + h * q + 3 * inner * h)
    attention = 2 * 2 * cfg["num_attention_heads"] * d * tokens * (tokens + 1) / 2
    return layers * (linear + attention) + 2 * h * cfg["vocab_size"]


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--layers", type=int, default=SIZES["num_hidden_layers"])
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    parser.add_argument("--only-decode", action="store_true",
                        help="time the decode steps only and print a short line (for profiling)")
    parser.add_argument("--only-prefill", action="store_true",
                        help="time the 2,048-token prefill only and print a short line (for profiling)")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace (candle, CPU); no cargo/rustc or maturin "
                          "offline, and its Python package binds only the cl100k tokenizer"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    args.warmup = max(args.warmup, 3)
    args.steps = max(1, min(args.steps, NEW_TOKENS - args.warmup - 1))

    import torch
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    from tokenizer_b200.kernels.ops import counter

    torch.cuda.set_device(0)
    cfg = dict(SIZES, num_hidden_layers=args.layers, max_window_layers=args.layers,
               architectures=["Qwen2ForCausalLM"], hidden_act="silu")
    config = tb.Qwen2Config.from_dict(cfg)
    pk = peaks()
    gen = torch.Generator().manual_seed(1234)

    def random_prompt(n):
        return torch.randint(0, config.vocab_size, (n,), generator=gen).tolist()

    with tempfile.TemporaryDirectory() as folder:
        tb.write_random_model(folder, config, seed=2)
        model = tb.load_model(folder, dtype="bfloat16", device="cuda:0")
    biggest = max(args.batch, 1 if (args.no_points or args.only_prefill) else 64)
    pool_tokens = max(biggest * (PROMPT_LEN + NEW_TOKENS + PAGE), PREFILL_TOKENS + PAGE)
    engine = tb.engine_for(model, pool_tokens, PAGE, max_requests=max(biggest, 1), share_prefixes=False)

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # ---- prefill of 2,048 tokens in one step ------------------------------------
    prefill_ms = []
    for rep in range(0 if args.only_decode else 3 + 5):
        cache = engine.cache.open(("prefill", rep))
        engine.cache.reserve(cache, PREFILL_TOKENS)
        entry = StepEntry(cache, random_prompt(PREFILL_TOKENS), [PREFILL_TOKENS - 1])
        torch.cuda.synchronize()
        start, stop = events()
        start.record()
        engine.step([entry])
        stop.record()
        torch.cuda.synchronize()
        if rep >= 3:
            prefill_ms.append(start.elapsed_time(stop))
        engine.cache.close(cache)
    prefill_best = sorted(prefill_ms)[len(prefill_ms) // 2] if prefill_ms else float("nan")
    if args.only_prefill:
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "layers": args.layers,
                          "ms": prefill_best, "tok_s": PREFILL_TOKENS / (prefill_best / 1e3)}))
        return 0
    prefill = {"value": PREFILL_TOKENS / (prefill_best / 1e3), "tokens": PREFILL_TOKENS,
               "ms": prefill_best,
               "frac": prefill_flops(cfg, args.layers, PREFILL_TOKENS) / (prefill_best / 1e3)
               / (pk["bf16_tflops"] * 1e12)}

    # ---- decode -----------------------------------------------------------------
    def decode_run(batch, steps, warmup, sample_clocks):
        caches = [engine.cache.open(("decode", batch, i)) for i in range(batch)]
        for lo in range(0, batch, 8):          # prompts in steps of up to 4,096 tokens
            group = caches[lo:lo + 8]
            for c in group:
                engine.cache.reserve(c, PROMPT_LEN)
            logits = engine.step([StepEntry(c, random_prompt(PROMPT_LEN), [PROMPT_LEN - 1])
                                  for c in group])
            first = engine.sampler.greedy(logits).tolist()
            for c, t in zip(group, first):
                c.next_token = t
        ids = engine.decode_steps([StepEntry(c, [c.next_token]) for c in caches], warmup)
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.start()
            time.sleep(0.25)
        torch.cuda.synchronize()
        launches = counter.launches
        start, stop = events()
        start.record()
        ids = engine.decode_steps([StepEntry(c, [t]) for c, t in zip(caches, ids[-1])], steps)
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop)
        launches = counter.launches - launches
        clock_record = clocks.stop() if clocks else None
        context = caches[0].length
        for c in caches:
            engine.cache.close(c)
        return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3),
                "launches": launches, "clocks": clock_record, "context_end": context}

    main_run = decode_run(args.batch, args.steps, args.warmup, not args.only_decode)
    if args.only_decode:
        print(json.dumps({"only": "decode", "batch": args.batch, "ms_per_step": main_run["ms_per_step"],
                          "tok_s": main_run["tok_s"], "gpu_launches": main_run["launches"]}))
        return 0
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = decode_run(b, min(args.steps, 64), 4, False)["tok_s"]

    mean_context = main_run["context_end"] - args.steps / 2
    step_bytes = weight_bytes(cfg, args.layers) + args.batch * mean_context * kv_bytes_per_token(cfg, args.layers)
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9

    # ---- the same through the Python entry point ----------------------------------
    from tokenizer_b200.engine.scheduler import Scheduler

    def through_scheduler(burst):
        """Decoding through the scheduler: host ids in, host ids out.  With burst 1
        every step copies its inputs to the device and its ids back."""
        prompts = [random_prompt(PROMPT_LEN) for _ in range(args.batch)]
        tokens = min(args.steps + args.warmup + burst, NEW_TOKENS)
        scheduler = Scheduler(engine, max_batch_size=args.batch, token_budget=8 * PROMPT_LEN,
                              decode_burst=burst)
        for p in prompts:
            scheduler.add_request(p, tb.GenerateParams(max_tokens=tokens))
        while any(len(r.context) == len(r.prompt) for r in scheduler.running) or scheduler.waiting:
            scheduler.step()                      # prompts, not timed
        while scheduler.stats.steps < args.warmup + 1:
            scheduler.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        sampled0, steps0 = scheduler.stats.tokens_sampled, scheduler.stats.steps
        while scheduler.has_work() and scheduler.stats.steps - steps0 + burst <= args.steps - 1:
            scheduler.step()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        steps = max(1, scheduler.stats.steps - steps0)
        value = (scheduler.stats.tokens_sampled - sampled0) / seconds
        scheduler.run()
        return value, steps

    e2e_value, e2e_steps = through_scheduler(1)
    h2d = engine.builder.last_bytes
    burst_value, burst_steps = through_scheduler(8)

    line = {
        "metric": "decode tok/s (Qwen2.5-0.5B sizes, batch %d, 512-token prompts)" % args.batch,
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": main_run["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": main_run["tok_s"] / 34.382, "dtype": "bf16",
        "data": "synthetic: random weights (seed 2), uniform random token ids",
        "config": {"model": "Qwen2.5-0.5B sizes", "layers": args.layers,
                   "layers_of_config": SIZES["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "global_batch": args.batch, "seq_len": PROMPT_LEN,
                   "new_tokens": NEW_TOKENS, "context_at_timing": int(mean_context),
                   "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "each step reads > 126 MB of weights (inputs larger than L2)",
                   "peaks": pk["source"]},
        "clocks": main_run["clocks"],
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * args.batch, "steps": e2e_steps,
                "note": "every step: its positions, slots and block tables from pinned host memory, its drawn "
                        "ids back to the host; a step's token ids reach it on the device, so the host reads "
                        "a draw while the next step runs"},
        "e2e_burst": {"value": burst_value, "unit": "tokens/s", "steps": burst_steps, "burst": 8,
                      "note": "8 greedy steps on the device between visits to the host: "
                              "one input copy and one read of 8 steps' ids per burst"},
        "gpu_launches": main_run["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
