"""The cache of a running engine: pages of keys and values, one block table per
request and group, and slots of fixed-size state.

Bookkeeping (which request holds which page) is the C++ `CacheManager`
(csrc/host/runtime.hpp); this class owns the device memory it indexes:

* one pool per *group* of (run-order entry, role) whose parts ask for the same kind
  of cache (kv heads, head size, window): `[entries, 2, pages, kv_heads, page,
  head_dim]`, k at index 0 and v at index 1.  A page id is valid in every entry
  of its group, as in the reference where one allocator serves every layer's
  pool (crates/ai-engine-candle/src/paged/engine.rs:70-73); groups with
  different needs have pools and block tables of their own.
* one state tensor per (entry, role) whose part asks for state: `[max_seqs, *shape]`,
  indexed by the request's slot and zeroed when the slot is given out.

Fresh pools are filled with NaN, so a read of a slot that was never written
shows in the logits.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..csrc.build import load_host_module
from ..parts.base import CacheNeed, KVRequest, LayerCache, StateRequest

_host = None


def host():
    """The compiled host runtime module (built on first use)."""
    global _host
    if _host is None:
        _host = load_host_module()
    return _host


@dataclass
class CacheGroup:
    request: KVRequest
    entries: List[Tuple[int, str]]     # (run-order index, role) that own a cache in this group
    page_size: int
    num_pages: int
    pool: Optional[torch.Tensor] = None    # [len(entries), 2, num_pages, K, page, d]

    @property
    def bytes_per_token(self) -> int:
        return 2 * len(self.entries) * self.request.kv_heads * self.request.head_dim


def group_requests(needs: Sequence[CacheNeed]):
    """Cache needs -> groups by what the parts ask for."""
    keys: Dict[KVRequest, List[Tuple[int, str]]] = {}
    for n in needs:
        if n.kv is not None and n.cache_from is None:
            keys.setdefault(n.kv, []).append((n.run, n.role))
    return list(keys.items())


class PagedCache:
    def __init__(self, requests: Sequence[CacheNeed], page_size: int, num_pages: int, max_seqs: int,
                 max_seq_len: int, dtype: torch.dtype, device="cuda", allocate: bool = True):
        """requests: `Model.cache_requests()`.  num_pages: pages of each group's pool.
        allocate=False keeps only the bookkeeping (tests without a device)."""
        self.requests = list(requests)
        self.page_size, self.num_pages = int(page_size), int(num_pages)
        self.max_seqs, self.max_seq_len = int(max_seqs), int(max_seq_len)
        self.dtype, self.device = dtype, torch.device(device)
        self.max_pages_per_seq = (self.max_seq_len + self.page_size - 1) // self.page_size
        self.groups: List[CacheGroup] = []
        self.where: Dict[Tuple[int, str], Tuple[int, int]] = {}       # (run, role) -> (group, index in group)
        self.writes: Dict[Tuple[int, str], bool] = {}
        for kv, entries in group_requests(self.requests):
            g = CacheGroup(kv, entries, self.page_size, self.num_pages)
            for j, e in enumerate(entries):
                self.where[e] = (len(self.groups), j)
                self.writes[e] = True
            self.groups.append(g)
        for n in self.requests:
            if n.cache_from is not None:
                if (n.cache_from, n.role) not in self.where:
                    raise ValueError(f"run order entry {n.run} ({n.role}) reads the cache of entry "
                                     f"{n.cache_from}, which has none")
                self.where[n.run, n.role] = self.where[n.cache_from, n.role]
                self.writes[n.run, n.role] = False
        self.roles: Dict[int, List[str]] = {}
        for n in self.requests:
            self.roles.setdefault(n.run, []).append(n.role)
        h = host()
        self.book = h.CacheManager([h.GroupSpec(g.page_size, g.num_pages, g.request.window)
                                    for g in self.groups], self.max_seqs, self.max_pages_per_seq)
        self.state: Dict[Tuple[int, str], torch.Tensor] = {}
        if allocate:
            for g in self.groups:
                r = g.request
                g.pool = torch.full((len(g.entries), 2, g.num_pages, r.kv_heads, g.page_size, r.head_dim),
                                    float("nan"), dtype=dtype, device=self.device)
            for n in self.requests:
                if n.state is not None:
                    self.state[n.run, n.role] = torch.zeros((self.max_seqs,) + tuple(n.state.shape),
                                                            dtype=n.state.dtype, device=self.device)

    # -- requests ---------------------------------------------------------------
    def admit(self) -> int:
        """A slot for a new request (-1: none free); its state starts at zero."""
        slot = self.book.admit()
        if slot >= 0:
            for t in self.state.values():
                t[slot].zero_()
        return slot

    def ensure(self, slot: int, n_tokens: int) -> bool:
        return self.book.ensure(slot, n_tokens)

    def advance(self, slot: int, computed: int) -> int:
        return self.book.advance(slot, computed)

    def finish(self, slot: int) -> None:
        self.book.finish(slot)

    def reset_state(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()

    # -- the step's view ----------------------------------------------------------
    def block_table_width(self, max_tokens: int) -> int:
        return max(1, (max_tokens + self.page_size - 1) // self.page_size)

    def part_cache(self, run_index: int, role: str, ctx) -> LayerCache:
        """What the part in `role` of run-order entry `run_index` gets of the cache in this step."""
        lc = LayerCache(state=self.state.get((run_index, role)))
        if (run_index, role) in self.where:
            g, j = self.where[run_index, role]
            grp = self.groups[g]
            lc.k_pages, lc.v_pages = grp.pool[j, 0], grp.pool[j, 1]
            lc.block_table = ctx.block_tables[g]
            lc.page_size = grp.page_size
            lc.writes = self.writes[run_index, role]
        return lc

    def layer_cache(self, run_index: int, ctx) -> Dict[str, LayerCache]:
        """role -> LayerCache for the parts of run-order entry `run_index` that asked for pages or state."""
        return {role: self.part_cache(run_index, role, ctx) for role in self.roles.get(run_index, ())}

    # -- accounting -----------------------------------------------------------------
    def kv_bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_token for g in self.groups) * es

    def stats(self) -> dict:
        return {f"group{g}": dict(pages=grp.num_pages, in_use=self.book.pages_in_use(g),
                                  high_water=self.book.high_water(g),
                                  allocations=self.book.total_allocations(g),
                                  window=grp.request.window)
                for g, grp in enumerate(self.groups)}
