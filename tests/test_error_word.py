"""The error word: a bounded wait on the device that runs out must fail the step on the host.
Here without a GPU: the word is an int the test owns; the GPU test that makes a wait run out
is in test_kernels_gpu.py."""
import ctypes

import pytest

from tokenizer_b200.kernels import ops


@pytest.fixture
def word(monkeypatch):
    value = ctypes.c_int(0)
    monkeypatch.setattr(ops, "_error_word", (value, 0))
    monkeypatch.setattr(ops, "_registered", {})
    return value


def test_a_clear_word_raises_nothing(word):
    ops.raise_if_error()
    assert ops.error_code() == 0


@pytest.mark.parametrize("code, library, text", [
    (3 * 16 + 2, "ffn_small_m", "between blocks"),
    (1 * 16 + 1, "gemm_tcgen05", "shared-memory barrier"),
    (2 * 16 + 2, "attention_tcgen05", "not aligned"),
    (4 * 16 + 1, "linear_stream", "shared-memory barrier"),
])
def test_a_set_word_raises_once_and_names_the_library(word, code, library, text):
    word.value = code
    with pytest.raises(ops.KernelError, match=library) as err:
        ops.raise_if_error("after step 7")
    assert text in str(err.value) and "after step 7" in str(err.value)
    assert word.value == 0
    ops.raise_if_error()          # cleared: the next check passes


def test_a_set_word_fails_the_scheduler_iteration(word):
    """An engine whose sampler finds the word set raises out of `Scheduler.step`; nothing is
    sampled from the wrong logits."""
    from fake_engine import FakeEngine
    from tokenizer_b200.engine.generate import GenerateParams
    from tokenizer_b200.engine.scheduler import Scheduler

    class Engine(FakeEngine):
        def sample(self, logits, temperature, top_p, uniform):
            ops.raise_if_error("found when a draw's ids were read")
            return super().sample(logits, temperature, top_p, uniform)

    s = Scheduler(Engine(num_pages=64), max_batch_size=2, token_budget=64)
    rid = s.add_request([1, 2, 3], GenerateParams(max_tokens=3))
    s.step()
    word.value = 3 * 16 + 1
    with pytest.raises(ops.KernelError, match="ffn_small_m"):
        s.step()
    assert rid not in s.finished
