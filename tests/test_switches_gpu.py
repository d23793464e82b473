"""Every environment switch that selects another kernel or launch order for the same
arithmetic gives the plain logits too: the alternates stay usable for comparisons.  The
switches are read at import, so each runs bin/trace_run in a process of its own."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import replay_util as ru
from tiny import random_ids

pytestmark = pytest.mark.gpu

SWITCHES = [
    {}, {"TOKB200_ATTENTION": "mma"}, {"TOKB200_FFN": "separate"}, {"TOKB200_QKV_NORM": "separate"},
    {"TOKB200_DECODE_MERGE": "scratch"}, {"TOKB200_STREAM": "0"}, {"TOKB200_PDL": "0"},
    {"TOKB200_GEMM": "library"}, {"TOKB200_QKV_ROPE": "fused"}, {"TOKB200_L2_PREFETCH": "1"},
    {"TOKB200_GEMM_PAIR": "0"}, {"TOKB200_LAYER": "fused"}, {"TOKB200_LAYER": "fused", "TOKB200_PDL": "0"},
    {"TOKB200_MIXED": "tiles"}, {"TOKB200_GEMM": "own"}, {"TOKB200_RING": "0"},
]


@pytest.fixture(scope="module")
def case(tmp_path_factory):
    """Sizes that reach the kernels the switches choose between: head size 64, an inner size
    in whole 128s, a vocabulary of enough rows for the streamed projection; two requests, a
    prompt of 300 tokens in one step and decoding beside a second request's portions."""
    import tokenizer_b200 as tb
    config = tb.Qwen2Config.from_dict(dict(
        architectures=["Qwen2ForCausalLM"], hidden_act="silu", num_hidden_layers=2, hidden_size=128,
        num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=256, vocab_size=9600,
        rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=1024,
        use_sliding_window=False, sliding_window=None, max_window_layers=2))
    folder = str(tmp_path_factory.mktemp("switches"))
    tb.write_random_model(folder, config, 12)
    a, b = random_ids(310, 9600, 5), random_ids(300, 9600, 6)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:300], "want": [0, 150, 299]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[300:301], "want": [0]},
                                     {"id": "b", "tokens": b[:256], "want": [255]}], "end": []}]
    for t in range(301, 306):
        steps.append({"step": len(steps), "entries": [
            {"id": "a", "tokens": a[t:t + 1], "want": [0]},
            {"id": "b", "tokens": b[256 + (t - 301):257 + (t - 301)], "want": [0]}], "end": []})
    steps[-1]["end"] = ["a", "b"]
    want = ru.reference_logits(folder, {"a": a[:306], "b": b[:261]})
    return folder, steps, want


@pytest.mark.parametrize("switch", SWITCHES, ids=lambda s: "+".join(f"{k}={v}" for k, v in s.items()) or "default")
def test_a_switch_changes_the_kernels_not_the_logits(case, switch, tmp_path):
    folder, steps, want = case
    cmd = [sys.executable, ru.TRACE_RUN, "--model", folder, "--dtype", "bfloat16", "--out", str(tmp_path),
           "--max-tokens", "1024", "--page-size", "16"]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=600,
                          env=dict(os.environ, **switch))
    assert proc.returncode == 0, proc.stderr[-3000:]
    vocab = 9600
    outputs = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        outputs[s["step"]] = np.fromfile(os.path.join(str(tmp_path), f"{s['step']}.f32"), dtype="<f4").reshape(wanted, vocab)
    got = ru.collect(steps, outputs)
    ru.compare(got, want, "bfloat16", f"switch {switch}")
