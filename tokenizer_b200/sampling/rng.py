"""The uniform draws of sampling.  A request with seed s draws, for its k-th
sampled token, u(s, k): a counter-based generator (splitmix64 over s and k), so
a request's draws do not depend on what else is in the batch or on how often it
was preempted.  The reference draws from the `rand` crate's StdRng
(qwen-infer/src/generate.rs:209, sample.rs:127); its stream is not reproduced,
so sampled ids agree with the reference in distribution, not id by id."""
from __future__ import annotations

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, counter: int) -> float:
    """A float in [0, 1) with 24 random bits, like `random::<f32>()`."""
    mixed = _splitmix64((_splitmix64(seed & _MASK) + counter * 0xD1342543DE82EF95) & _MASK)
    return (mixed >> 40) / float(1 << 24)
