"""The device side of the cache: one pool of pages per group, one state arena
per call that declares state, and the bindings handed to the mixers."""
from __future__ import annotations

from typing import List

import torch

from ..parts.base import CacheBinding, Runtime
from .manager import CachePlan, RequestCache


class DeviceCache(CachePlan):
    """`CachePlan` plus the memory.  Pool of group g:
    [calls in the group, 2 (keys, values), pages * page_size, kv_heads, head_dim]
    in the compute dtype; a token's keys of one call lie at row
    page * page_size + offset."""

    def __init__(self, needs, num_pages: int, page_size: int, max_requests: int,
                 runtime: Runtime, share_prefixes: bool = False):
        super().__init__(needs, num_pages, page_size, max_requests, share_prefixes)
        self.runtime = runtime
        self.pools: List[torch.Tensor] = []
        for layout in self.groups:
            self.pools.append(torch.zeros(
                (len(layout.calls), 2, num_pages * page_size, layout.kv_heads, layout.head_dim),
                dtype=runtime.dtype, device=runtime.device))
        self.states = {}
        for call in self.state_calls:
            self.states[call] = torch.zeros(
                (max_requests,) + tuple(needs[call].state.shape), dtype=torch.float32,
                device=runtime.device)
        self._needs = needs

    def on_open(self, cache: RequestCache) -> None:
        for arena in self.states.values():
            arena[cache.state_slot].zero_()

    def bindings(self, order) -> List[CacheBinding]:
        """One binding per call of the order."""
        out = []
        for at, call in enumerate(order):
            source = at if call.cache is None else call.cache
            group = self.group_of_call[source]
            binding = CacheBinding(writes=call.cache is None)
            if group is not None:
                layer = self.groups[group].calls.index(source)
                binding.group = group
                binding.k_pool = self.pools[group][layer, 0]
                binding.v_pool = self.pools[group][layer, 1]
            binding.state = self.states.get(source)
            out.append(binding)
        return out

    def bytes_per_token(self) -> int:
        size = torch.empty((), dtype=self.runtime.dtype).element_size()
        return sum(len(g.calls) * 2 * g.kv_heads * g.head_dim * size for g in self.groups)
