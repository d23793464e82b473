"""The kernels at the widths of real checkpoints (Qwen2.5-0.5B, the benchmark's; 1.5B and 7B with
head size 128, the latter with four key/value heads and an untied head), a few
layers each: tiny configurations do not reach the tcgen05 tiles of 128, the streamed vocabulary
projection or the fused feed-forward at their real shapes.  One plain float32 forward on the CPU
over one long id sequence serves every request, because each request's prompt is a beginning of it."""
import pytest
import torch

import plain_qwen2 as plain
from tiny import random_ids

pytestmark = pytest.mark.gpu


WIDTHS = {
    "0.5B": dict(num_hidden_layers=3, hidden_size=896, num_attention_heads=14, num_key_value_heads=2,
                 intermediate_size=4864, vocab_size=151936, tie_word_embeddings=True),
    "1.5B": dict(num_hidden_layers=2, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2,
                 intermediate_size=8960, vocab_size=151936, tie_word_embeddings=True),
    # the 7B widths with a third of its vocabulary (the two tables are most of a one-layer model)
    "7B": dict(num_hidden_layers=1, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, vocab_size=50021, tie_word_embeddings=False),
}


@pytest.mark.parametrize("widths", list(WIDTHS))
def test_prompt_and_decoding_at_real_widths(tmp_path_factory, widths):
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    sizes = WIDTHS[widths]
    config = tb.Qwen2Config.from_dict(dict(
        sizes, architectures=["Qwen2ForCausalLM"], hidden_act="silu",
        rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=4096,
        use_sliding_window=False, sliding_window=4096, max_window_layers=sizes["num_hidden_layers"]))
    path = str(tmp_path_factory.mktemp("real_sizes"))
    # Attention is left as flat as random weights make it: sharpened fourfold, the rounding of q
    # and k to bfloat16 alone moves these logits by 4 % of their largest (0.13; the same with the
    # mma.sync attention and with library products), which would drown what this test looks for.
    tb.write_random_model(path, config, 9)
    cfg, w = plain.load_folder(path)
    ids = random_ids(300, config.vocab_size, 77)
    want = plain.all_logits(cfg, w, ids)                      # [300, vocab]: row t = logits after ids[:t + 1]
    bound = 2e-2 * float(want.abs().max())
    # the 32-bit path first: the same logic at these widths, to 1e-4
    exact = tb.engine_for(tb.load_model(path, dtype="float32"), 320, 16, max_requests=1)
    cache = exact.cache.open("exact")
    exact.cache.reserve(cache, 256)
    got = exact.step([StepEntry(cache, ids[:256], [0, 100, 255])]).cpu()
    off = float((got - want[[0, 100, 255]]).abs().max())
    print(f"{widths}: largest logit {float(want.abs().max()):.3f}, 32-bit path off by {off:.2e}")
    assert off <= 1e-4
    del exact
    torch.cuda.empty_cache()
    model = tb.load_model(path, dtype="bfloat16")
    engine = tb.engine_for(model, 8 * 320, 16, max_requests=8)

    def check(got, rows, what):
        err = (got.float().cpu() - want[rows]).abs().max(dim=1).values
        print(f"{widths}: {what}: off by {float(err.max()):.4f} of {bound:.4f} allowed")
        assert float(err.max()) <= bound, f"{what}: row {rows[int(err.argmax())]} is off by {float(err.max())}"

    # a prompt of 256 tokens three times over (run plainly, captured, replayed), then single tokens
    for use in range(3):
        cache = engine.cache.open(("whole", use))
        engine.cache.reserve(cache, 256)
        check(engine.step([StepEntry(cache, ids[:256], [0, 100, 255])]), [0, 100, 255], f"prompt, use {use}")
        if use < 2:
            engine.cache.close(cache)
    for t in range(256, 262):
        engine.cache.reserve(cache, 1)
        check(engine.step([StepEntry(cache, [ids[t]], [0])]), [t], f"decode alone at {t}")
    engine.cache.close(cache)
    # eight requests whose prompts are beginnings of the same sequence, then decoded together
    lengths = [200 + 7 * i for i in range(8)]
    caches = [engine.cache.open(("r", i)) for i in range(8)]
    for c, n in zip(caches, lengths):
        engine.cache.reserve(c, n)
    check(engine.step([StepEntry(c, ids[:n], [n - 1]) for c, n in zip(caches, lengths)]),
          [n - 1 for n in lengths], "eight prompts in one step")
    for step in range(4):
        for c in caches:
            engine.cache.reserve(c, 1)
        rows = [n + step for n in lengths]
        check(engine.step([StepEntry(c, [ids[r]], [0]) for c, r in zip(caches, rows)]), rows,
              f"eight decoded together, step {step}")
    # the same eight through steps that stay on the device: ids must be those of the plain argmax
    # where it leads clearly
    drawn = engine.decode_steps([StepEntry(c, [ids[n + 4]]) for c, n in zip(caches, lengths)], 1)
    top2 = torch.topk(want[[n + 4 for n in lengths]], 2, dim=-1).values
    for i, n in enumerate(lengths):
        if float(top2[i, 0] - top2[i, 1]) > 2 * bound:
            assert drawn[0][i] == int(want[n + 4].argmax())
