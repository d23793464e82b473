"""The command line, in the manner of the reference's `qwen-infer`
(qwen-infer/src/main.rs:12-148): the same options with the same meanings and
defaults, text on standard output, ids and timings on standard error.  The
model comes from a local folder; a prompt is text when the folder has a
tokenizer.json, or ids with --ids.

Beyond the reference's options: several prompts (positional arguments or `--ids` given more
than once) run together through the scheduler, and the scheduler's and the cache's sizes can
be set: --num-pages N (pages of the cache; default: room for every prompt to its end),
--page-size N (tokens a page, default 16), --max-batch-size N (requests that run together,
default 8 as the reference's server: qwen-server/src/lib.rs:47-55), --token-budget N (tokens a
step may run: prompts are cut into portions under it; default 2048).  --num-blocks,
--block-size and --prefill-chunk are other names for the first, second and fourth.  With a
small --num-pages requests are preempted and recomputed; the ids do not change."""
from __future__ import annotations

import os
import sys
import tempfile
import time

USAGE = ("usage: qwen-infer [--max-tokens N] [--temperature T] [--top-p P] [--seed N] "
         "[--stop STRING]... [--model DIR | --random-weights CONFIG.json] [--dtype bfloat16|float32] "
         "[--num-pages N] [--page-size N] [--max-batch-size N] [--token-budget N] "
         "[--ids 1,2,3]... [<prompt>]...")


class UsageError(Exception):
    pass


def parse_args(argv):
    args = dict(prompts=[], ids=[], max_tokens=20, temperature=0.0, top_p=1.0, seed=0, stop=[],
                model=os.environ.get("QWEN_INFER_MODEL"), random_weights=None, dtype="bfloat16",
                weights_seed=0, device="cuda:0", num_pages=None, page_size=16, max_batch_size=8,
                token_budget=2048)
    it = iter(argv)

    def value(flag):
        try:
            return next(it)
        except StopIteration:
            raise UsageError(f"{flag} needs a value") from None

    for arg in it:
        if arg in ("--help", "-h"):
            args["help"] = True
        elif arg == "--max-tokens":
            args["max_tokens"] = _number(int, value(arg), arg)
        elif arg == "--temperature":
            args["temperature"] = _number(float, value(arg), arg)
        elif arg == "--top-p":
            args["top_p"] = _number(float, value(arg), arg)
        elif arg == "--seed":
            args["seed"] = _number(int, value(arg), arg)
        elif arg == "--stop":
            args["stop"].append(value(arg))
        elif arg == "--model":
            args["model"] = value(arg)
        elif arg == "--random-weights":
            args["random_weights"] = value(arg)
        elif arg == "--weights-seed":
            args["weights_seed"] = _number(int, value(arg), arg)
        elif arg == "--dtype":
            args["dtype"] = value(arg)
        elif arg == "--device":
            args["device"] = value(arg)
        elif arg == "--ids":
            args["ids"].append([_number(int, v, arg) for v in value(arg).split(",") if v.strip()])
        elif arg in ("--num-pages", "--num-blocks"):
            args["num_pages"] = _positive(value(arg), arg)
        elif arg in ("--page-size", "--block-size"):
            args["page_size"] = _positive(value(arg), arg)
        elif arg == "--max-batch-size":
            args["max_batch_size"] = _positive(value(arg), arg)
        elif arg in ("--token-budget", "--prefill-chunk"):
            args["token_budget"] = _positive(value(arg), arg)
        elif arg.startswith("-") and arg != "-":
            raise UsageError(f"unknown argument {arg}")
        else:
            args["prompts"].append(arg)
    if args["prompts"] and args["ids"]:
        raise UsageError("prompts come as text or as --ids, not both")
    return args


def _positive(text, flag):
    n = _number(int, text, flag)
    if n < 1:
        raise UsageError(f"{flag} {text}: must be at least 1")
    return n


def _number(kind, text, flag):
    try:
        return kind(text)
    except ValueError:
        raise UsageError(f"{flag} {text}: not a number") from None


def main(argv=None) -> int:
    try:
        args = parse_args(sys.argv[1:] if argv is None else argv)
    except UsageError as err:
        print(err, file=sys.stderr)
        print(USAGE, file=sys.stderr)
        return 2
    if args.get("help"):
        print(USAGE, file=sys.stderr)
        return 0
    if not args["prompts"] and not args["ids"]:
        print(USAGE, file=sys.stderr)
        return 1

    import json

    import tokenizer_b200 as tb
    from tokenizer_b200.text import ByteLevelBPE

    scratch = None
    folder = args["model"]
    if args["random_weights"]:
        with open(args["random_weights"]) as fh:
            config = tb.config.config_from_dict(json.load(fh))
        scratch = tempfile.TemporaryDirectory()
        folder = tb.write_random_model(scratch.name, config, args["weights_seed"])
    if not folder:
        print("no model: give --model DIR (or set QWEN_INFER_MODEL), or --random-weights CONFIG.json",
              file=sys.stderr)
        return 1

    tokenizer = None
    tokenizer_path = os.path.join(folder, "tokenizer.json")
    if os.path.exists(tokenizer_path):
        tokenizer = ByteLevelBPE.from_file(tokenizer_path)
    if args["ids"]:
        prompts = args["ids"]
    elif tokenizer is None:
        print(f"{folder} has no tokenizer.json: give the prompt as --ids 1,2,3", file=sys.stderr)
        return 1
    else:
        prompts = [tokenizer.encode(text) for text in args["prompts"]]
    if any(not ids for ids in prompts):
        print("prompt encoded to no tokens", file=sys.stderr)
        return 1
    several = len(prompts) > 1
    for index, ids in enumerate(prompts):
        label = f"prompt {index} ids" if several else "prompt ids"
        print(f"{label} ({len(ids)}): {ids}", file=sys.stderr)

    params = tb.GenerateParams(max_tokens=args["max_tokens"], temperature=args["temperature"],
                               top_p=args["top_p"], seed=args["seed"],
                               eos=tb.load_eos_token_ids(folder), stop=args["stop"])
    print(f"max_tokens {params.max_tokens} temperature {params.temperature} top_p {params.top_p} "
          f"seed {params.seed} eos {list(params.eos)}", file=sys.stderr)
    scheduler = None
    try:
        params.validate()
        model = tb.load_model(folder, dtype=args["dtype"], device=args["device"])
        page = args["page_size"]
        pages = args["num_pages"]
        if pages is None:
            pages = sum(-(-(len(ids) + params.max_tokens + 1) // page) for ids in prompts)
        batch = min(args["max_batch_size"], len(prompts))
        engine = tb.Engine(model, num_pages=pages, page_size=page, max_requests=batch,
                           share_prefixes=True)
        started = time.perf_counter()
        token_bytes = (lambda t: tokenizer.decode_bytes([t])) if tokenizer else None
        scheduler = tb.Scheduler(engine, max_batch_size=batch, token_budget=args["token_budget"])
        ids = [scheduler.add_request(p, params, token_bytes) for p in prompts]
        finished = scheduler.run()
        results = [finished[i] for i in ids]
        elapsed = time.perf_counter() - started
    except (ValueError, RuntimeError) as err:
        print(f"error: {err}", file=sys.stderr)
        return 1
    finally:
        if scratch is not None:
            scratch.cleanup()
    status = 0
    for index, generated in enumerate(results):
        tag = f"[{index}] " if several else ""
        if generated.reason == tb.StopReason.FAILED:
            print(f"{tag}error: {generated.error}", file=sys.stderr)
            print("")
            status = 1
            continue
        print(generated.text if tokenizer else " ".join(str(t) for t in generated.tokens))
        print(f"{tag}generated ids: {generated.tokens}", file=sys.stderr)
        print(f"{tag}stop: {generated.reason.name}", file=sys.stderr)
        n = len(generated.tokens)
        if n == 0 or generated.decode == 0.0:
            print(f"{tag}prefill {generated.prefill:.4f} s, decode {generated.decode:.4f} s, {n} tokens "
                  f"(KV cache, total {elapsed:.4f} s)", file=sys.stderr)
        else:
            print(f"{tag}prefill {generated.prefill:.4f} s, decode {generated.decode:.4f} s, "
                  f"{n / generated.decode:.4f} tok/s ({n} tokens, KV cache, total {elapsed:.4f} s)",
                  file=sys.stderr)
        if generated.reason == tb.StopReason.EOS:
            print(f"{tag}stopped on eos before max_tokens", file=sys.stderr)
    if several or args["num_pages"] is not None:
        stats = scheduler.stats
        print(f"scheduler: {stats.steps} steps, most running {stats.max_running}, preemptions "
              f"{stats.preemptions}, most pages held {stats.peak_pages} of {pages}, shared prefix "
              f"tokens {stats.shared_prefix_tokens}", file=sys.stderr)
    return status


if __name__ == "__main__":
    sys.exit(main())
