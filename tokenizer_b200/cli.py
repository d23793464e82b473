"""The command line, in the manner of the reference's `qwen-infer`
(qwen-infer/src/main.rs:12-148): the same options with the same meanings and
defaults, text on standard output, ids and timings on standard error.  The
model comes from a local folder; a prompt is text when the folder has a
tokenizer.json, or ids with --ids."""
from __future__ import annotations

import os
import sys
import tempfile
import time

USAGE = ("usage: qwen-infer [--max-tokens N] [--temperature T] [--top-p P] [--seed N] "
         "[--stop STRING]... [--model DIR | --random-weights CONFIG.json] [--dtype bfloat16|float32] "
         "[--ids 1,2,3 | <prompt>]")


class UsageError(Exception):
    pass


def parse_args(argv):
    args = dict(prompt=None, ids=None, max_tokens=20, temperature=0.0, top_p=1.0, seed=0, stop=[],
                model=os.environ.get("QWEN_INFER_MODEL"), random_weights=None, dtype="bfloat16",
                weights_seed=0, device="cuda:0")
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
            args["ids"] = [_number(int, v, arg) for v in value(arg).split(",") if v.strip()]
        elif arg.startswith("-") and arg != "-":
            raise UsageError(f"unknown argument {arg}")
        else:
            if args["prompt"] is not None:
                raise UsageError(f"only one prompt is accepted (got {arg!r} as well)")
            args["prompt"] = arg
    return args


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
    if (args["prompt"] is None) == (args["ids"] is None):
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
    if args["ids"] is not None:
        prompt_ids = args["ids"]
    elif tokenizer is None:
        print(f"{folder} has no tokenizer.json: give the prompt as --ids 1,2,3", file=sys.stderr)
        return 1
    else:
        prompt_ids = tokenizer.encode(args["prompt"])
    if not prompt_ids:
        print("prompt encoded to no tokens", file=sys.stderr)
        return 1
    print(f"prompt ids ({len(prompt_ids)}): {prompt_ids}", file=sys.stderr)

    params = tb.GenerateParams(max_tokens=args["max_tokens"], temperature=args["temperature"],
                               top_p=args["top_p"], seed=args["seed"],
                               eos=tb.load_eos_token_ids(folder), stop=args["stop"])
    print(f"max_tokens {params.max_tokens} temperature {params.temperature} top_p {params.top_p} "
          f"seed {params.seed} eos {list(params.eos)}", file=sys.stderr)
    try:
        params.validate()
        model = tb.load_model(folder, dtype=args["dtype"], device=args["device"])
        started = time.perf_counter()
        token_bytes = (lambda t: tokenizer.decode_bytes([t])) if tokenizer else None
        generated = tb.generate(model, prompt_ids, params, token_bytes)
        elapsed = time.perf_counter() - started
    except (ValueError, RuntimeError) as err:
        print(f"error: {err}", file=sys.stderr)
        return 1
    finally:
        if scratch is not None:
            scratch.cleanup()
    print(generated.text if tokenizer else " ".join(str(t) for t in generated.tokens))
    print(f"generated ids: {generated.tokens}", file=sys.stderr)
    print(f"stop: {generated.reason.name}", file=sys.stderr)
    n = len(generated.tokens)
    if n == 0 or generated.decode == 0.0:
        print(f"prefill {generated.prefill:.4f} s, decode {generated.decode:.4f} s, {n} tokens "
              f"(KV cache, total {elapsed:.4f} s)", file=sys.stderr)
    else:
        print(f"prefill {generated.prefill:.4f} s, decode {generated.decode:.4f} s, "
              f"{n / generated.decode:.4f} tok/s ({n} tokens, KV cache, total {elapsed:.4f} s)",
              file=sys.stderr)
    if generated.reason == tb.StopReason.EOS:
        print("stopped on eos before max_tokens", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
