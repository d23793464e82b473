"""The Python entry point, in the reference library's names
(qwen-infer/src/lib.rs:14-24, generate.rs:75-145): `load_model`, `generate`,
`generate_with`, `greedy_tokens`, `load_eos_token_ids`, with token ids in and
out on the host.  `generate_batch` runs several prompts through the scheduler
at once."""
from __future__ import annotations

import json
import os
from typing import Callable, List, Optional, Sequence, Union

from .engine.generate import Control, Generated, GenerateParams, StopReason
from .engine.scheduler import Scheduler
from .engine.step import Engine, load_model, random_model

__all__ = ["Control", "Engine", "Generated", "GenerateParams", "StopReason", "generate",
           "generate_batch", "generate_with", "greedy_tokens", "load_eos_token_ids", "load_model",
           "engine_for", "random_model"]


def load_eos_token_ids(path: str) -> List[int]:
    """`eos_token_id` of a generation_config.json: one id or a list
    (qwen-infer/src/lib.rs:84-113).  A folder without the file has none."""
    if os.path.isdir(path):
        path = os.path.join(path, "generation_config.json")
    if not os.path.exists(path):
        return []
    with open(path) as fh:
        value = json.load(fh).get("eos_token_id")
    if value is None:
        return []
    if isinstance(value, int) and not isinstance(value, bool):
        return [value]
    if isinstance(value, list) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
        return list(value)
    raise ValueError(f"{path}: eos_token_id must be an integer or a list of integers")


def engine_for(model, tokens: int, page_size: int = 16, max_requests: int = 64,
               share_prefixes: bool = True) -> Engine:
    """An engine whose pool holds `tokens` tokens (rounded up to whole pages
    per request by the caller)."""
    pages = max(1, -(-int(tokens) // page_size))
    return Engine(model, num_pages=pages, page_size=page_size, max_requests=max_requests,
                  share_prefixes=share_prefixes)


def generate_batch(model_or_engine, prompts: Sequence[Sequence[int]],
                   params: Union[GenerateParams, Sequence[GenerateParams]],
                   token_bytes: Optional[Callable[[int], bytes]] = None,
                   on_chunk: Optional[Callable[[int, str], Control]] = None,
                   max_batch_size: int = 64, token_budget: int = 2048,
                   page_size: int = 16, decode_burst: int = 1) -> List[Generated]:
    """Run every prompt to its end with continuous batching; results in the
    order of `prompts`.  `on_chunk(index, text)` may return Control.STOP.
    `decode_burst` > 1 lets greedy decoding run that many steps on the device
    between visits to the host (text then arrives in pieces of that many ids)."""
    if isinstance(params, GenerateParams):
        params = [params] * len(prompts)
    if len(params) != len(prompts):
        raise ValueError("one GenerateParams for all prompts, or one each")
    if hasattr(model_or_engine, "step") and hasattr(model_or_engine, "cache"):
        engine = model_or_engine
    else:
        need = sum((len(p) + q.max_tokens + page_size) // page_size * page_size
                   for p, q in zip(prompts, params))
        engine = engine_for(model_or_engine, need, page_size,
                            max_requests=max(1, min(max_batch_size, len(prompts))))
    scheduler = Scheduler(engine, max_batch_size=min(max_batch_size, engine.cache.max_requests),
                          token_budget=token_budget, decode_burst=decode_burst)
    ids = []
    for index, (prompt, p) in enumerate(zip(prompts, params)):
        callback = (lambda text, index=index: on_chunk(index, text)) if on_chunk else None
        ids.append(scheduler.add_request(prompt, p, token_bytes, callback))
    results = scheduler.run()
    return [results[i] for i in ids]


def generate_with(model_or_engine, prompt: Sequence[int], params: GenerateParams,
                  token_bytes: Optional[Callable[[int], bytes]] = None,
                  on_chunk: Optional[Callable[[str], Control]] = None) -> Generated:
    """Prefill `prompt`, then sample up to `params.max_tokens` ids, one cached
    step each; `on_chunk` sees every piece of text that is safe to show."""
    callback = (lambda _index, text: on_chunk(text)) if on_chunk else None
    result = generate_batch(model_or_engine, [prompt], params, token_bytes, callback,
                            max_batch_size=1)[0]
    if result.reason == StopReason.FAILED:
        raise RuntimeError(result.error)
    return result


def generate(model_or_engine, prompt: Sequence[int], params: GenerateParams,
             token_bytes: Optional[Callable[[int], bytes]] = None) -> Generated:
    return generate_with(model_or_engine, prompt, params, token_bytes, None)


def greedy_tokens(model_or_engine, prompt: Sequence[int], n: int) -> List[int]:
    """`n` greedy ids after `prompt` (qwen-infer/src/lib.rs:120-133)."""
    return generate(model_or_engine, prompt, GenerateParams.greedy(n)).tokens
