"""Greedy, temperature and nucleus sampling on the device, one row of float32
logits per request (reference: qwen-infer/src/sample.rs:43-137).  temperature 0
is argmax with ties to the lower id and ignores top_p; otherwise weights
exp((l - max)/T), candidates by logit descending, the shortest prefix whose
share reaches top_p, and one draw u scaled by the kept weight."""
from __future__ import annotations

import math
from typing import List, Sequence

import torch

from ..kernels import ops


def validate_sampling(temperature: float, top_p: float) -> None:
    """sample.rs:77-88 and generate.rs:409-424."""
    if not math.isfinite(temperature):
        raise ValueError(f"temperature {temperature} is not finite")
    if temperature < 0:
        raise ValueError(f"temperature {temperature} is negative")
    if not math.isfinite(top_p):
        raise ValueError(f"top_p {top_p} is not finite")
    if top_p < 0:
        raise ValueError(f"top_p {top_p} is negative")


class PendingIds:
    """Ids on their way from the device; one outstanding draw per sampler at a time.
    `device_ids` (int32, one a row) can feed the next step before the host has read them."""

    def __init__(self, host, done, device_ids=None):
        self._host, self._done = host, done
        self.device_ids = device_ids

    def result(self) -> List[int]:
        if self._host is None:
            return []
        self._done.synchronize()
        # the step that made these logits has finished: had one of its bounded waits run out,
        # the ids would come from wrong logits
        ops.raise_if_error("found when a draw's ids were read")
        return self._host.tolist()


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._pinned = None
        self.scratch = ops.ScratchSpace()       # the greedy choice's partial results and counters

    def sample(self, logits: torch.Tensor, temperature: Sequence[float], top_p: Sequence[float],
               uniform: Sequence[float]) -> List[int]:
        """One id per row.  All-greedy batches skip the parameter upload."""
        return self.sample_launch(logits, temperature, top_p, uniform).result()

    def sample_launch(self, logits: torch.Tensor, temperature: Sequence[float],
                      top_p: Sequence[float], uniform: Sequence[float]) -> "PendingIds":
        """Start the draw and the copy of the ids to pinned host memory; `result()` waits for
        them.  What the host does in between runs beside the device."""
        n = logits.shape[0]
        if n == 0:
            return PendingIds(None, None)
        if logits.shape[1] == 0:
            raise ValueError("no logits to sample")
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        with ops.scratch_scope(self.scratch):
            if all(t == 0 for t in temperature):
                ops.sample(logits, None, None, None, out)
            else:
                params = torch.tensor([list(temperature), list(top_p), list(uniform)],
                                      dtype=torch.float32).to(self.device, non_blocking=True)
                ops.sample(logits, params[0], params[1], params[2], out)
        if self._pinned is None or self._pinned.numel() < n:
            self._pinned = torch.empty(max(n, 256), dtype=torch.int32, pin_memory=True)
        host = self._pinned[:n]
        host.copy_(out, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return PendingIds(host, done, out)

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        with ops.scratch_scope(self.scratch):
            ops.sample(logits, None, None, None, out)
        return out
