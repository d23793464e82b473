"""Helpers that drive bin/trace_run the way a user does (a subprocess, steps on
standard input) and compare what it writes with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

import plain_qwen2 as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# Largest |engine - plain| allowed on a logit.  float32: the bound the reference
# holds its own paths to (model.rs:1471, 1623, 1778).  bfloat16: operands carry 8
# bits of mantissa (relative step 2^-8); through a few layers the rounding of
# activations and of the cache adds up to well under 2% of the largest logit.
F32_TOL = 1e-4
BF16_REL_TOL = 2e-2


def rounded64(n):
    return (n + 63) // 64 * 64


def run_trace(folder, dtype, steps, out_dir, max_tokens, page_size, timeout=600, share=False,
              adopted=None):
    """Feed `steps` (list of dicts) and return {step: array [wanted, vocab]}.  With `share`
    the program may share pages between requests; `adopted` (a dict) is then filled with
    {request: tokens it took over instead of computing}."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
    if share:
        cmd.append("--share-prefixes")
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, f"trace_run failed:\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert [d.split()[1] for d in done] == [str(s["step"]) for s in steps], proc.stdout[-2000:]
    if adopted is not None:
        for line in proc.stdout.splitlines():
            if line.startswith("adopted "):
                adopted[line.split()[1]] = int(line.split()[2])
    vocab = json.load(open(os.path.join(folder, "config.json")))["vocab_size"]
    out = {}
    for s in steps:
        wanted = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if wanted:
            data = np.fromfile(path, dtype="<f4")
            assert data.size == wanted * vocab, f"step {s['step']}: {data.size} floats"
            out[s["step"]] = data.reshape(wanted, vocab)
        else:
            assert not os.path.exists(path)
    return out


def collect(steps, outputs):
    """{request: {position: logits row}} from the steps and what was written."""
    held = {}
    got = {}
    for s in steps:
        row = 0
        for e in s["entries"]:
            start = held.get(e["id"], 0)
            for w in e.get("want", []):
                got.setdefault(e["id"], {})[start + w] = outputs[s["step"]][row]
                row += 1
            held[e["id"]] = start + len(e["tokens"])
        for name in s.get("end", []):
            held.pop(name, None)
    return got


def reference_logits(folder, requests):
    """{request: array [len, vocab]} from the plain implementation."""
    cfg, weights = plain.load_folder(folder)
    return {name: plain.all_logits(cfg, weights, ids).numpy() for name, ids in requests.items()}


def compare(got, want, dtype, what):
    """Every collected row against the plain implementation; on a failure name
    the first wrong (request, position)."""
    worst = 0.0
    for name in sorted(got):
        ref = want[name]
        scale = float(np.abs(ref).max())
        tol = F32_TOL if dtype == "float32" else BF16_REL_TOL * scale
        for position in sorted(got[name]):
            err = float(np.abs(got[name][position] - ref[position]).max())
            assert np.isfinite(got[name][position]).all(), f"{what}: {name}[{position}] not finite"
            assert err <= tol, (
                f"{what} ({dtype}): first wrong logits at request {name!r} position {position}: "
                f"max |diff| {err:.3e} > {tol:.3e} (largest logit {scale:.3f})")
            worst = max(worst, err)
    return worst


# ---- ways of cutting the same requests ------------------------------------------
def steps_whole(requests, want_all=True):
    steps = []
    for at, (name, ids) in enumerate(requests.items()):
        want = list(range(len(ids))) if want_all else [len(ids) - 1]
        steps.append({"step": at, "entries": [{"id": name, "tokens": ids, "want": want}],
                      "end": [name]})
    return steps


def steps_decode_tail(requests, tail=32):
    steps, at = [], 0
    for name, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append({"step": at, "entries": [{"id": name, "tokens": ids[:head],
                                              "want": [head - 1]}], "end": []})
        at += 1
        for p in range(head, len(ids)):
            steps.append({"step": at, "entries": [{"id": name, "tokens": [ids[p]], "want": [0]}],
                          "end": [name] if p == len(ids) - 1 else []})
            at += 1
        if head == len(ids):
            steps[-1]["end"] = [name]
    return steps


def steps_portions(requests, sizes=(2, 7, 3, 16, 2, 33, 5, 2, 64, 9)):
    steps, at = [], 0
    for name, ids in requests.items():
        done, k = 0, 0
        while done < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - done)
            k += 1
            last = done + n == len(ids)
            steps.append({"step": at, "entries": [{"id": name, "tokens": ids[done:done + n],
                                                  "want": list(range(n))}],
                          "end": [name] if last else []})
            done += n
            at += 1
    return steps


def steps_mixed(requests, max_live=4, prompt_fraction=0.6, portion=(11, 2, 24, 5, 17),
                seed=0, share=None, page=16):
    """Up to `max_live` requests at a time: a request's first part goes in
    portions of changing size, the rest token by token; each step carries the
    portions of some beside the single tokens of others, one request is left out
    of a step now and then.  Returns the steps and the most tokens (each request
    rounded up to 64) that were live at once.

    `share` = {adopter: (donor, n)}: the adopter's first n tokens equal the donor's.  The
    donor's pages are published in the step that completes its first n tokens; the adopter
    starts only after that, while the donor is still live, with an entry that asks to adopt
    and wants logits only behind the whole pages it takes over.  Returns also
    {adopter: tokens it is expected to adopt}."""
    rng = np.random.RandomState(seed)
    share = share or {}
    waiting = list(requests.items())
    live = []   # [name, ids, done, prompt_len, k]
    steps, at, peak = [], 0, 0
    published = set()
    expect = {}
    while waiting or live:
        while waiting and len(live) < max_live:
            name = waiting[0][0]
            if name in share and share[name][0] not in published:
                assert any(item[0] == share[name][0] for item in live), "the donor must run first"
                break                      # its donor has not published yet
            name, ids = waiting.pop(0)
            live.append([name, ids, 0, max(2, int(len(ids) * prompt_fraction)), 0])
        entries, ended, publish = [], [], []
        for item in live:
            name, ids, done, prompt_len, k = item
            if len(live) > 1 and rng.rand() < 0.15:
                continue   # left out of this step
            if done < prompt_len:
                n = min(portion[(k + len(name)) % len(portion)], prompt_len - done)
            else:
                n = 1
            entry = {"id": name}
            first = 0
            if done == 0 and name in share:
                n = share[name][1] + 1 + n             # the shared beginning and a little more
                first = min(share[name][1], n - 1) // page * page
                expect[name] = first
                entry["adopt"] = True
            n = min(n, len(ids) - done)
            entry.update(tokens=ids[done:done + n], want=list(range(first, n)))
            entries.append(entry)
            item[2] += n
            item[4] += 1
            if item[2] == len(ids):
                ended.append(name)
            most = max([n_shared for donor, n_shared in share.values() if donor == name], default=None)
            if most is not None and name not in published and item[2] >= most:
                published.add(name)             # once all that its adopters will look for is in place
                publish.append(name)
        peak = max(peak, sum(rounded64(item[2]) for item in live))
        if entries:
            steps.append({"step": at, "entries": entries, "end": ended})
            if publish:
                steps[-1]["publish"] = publish
            at += 1
        live = [item for item in live if item[0] not in ended]
    if share:
        return steps, peak, expect
    return steps, peak
