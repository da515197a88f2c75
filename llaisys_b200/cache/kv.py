"""Device storage of the cache and the per-step views the mixers get.

Storage is paged: a page holds `PAGE` consecutive tokens of one sequence, for every user of its
group, laid out [page, kv head, token, dim] so that one head's keys of a page are contiguous.
A user is one mixer of one entry of the model's run order.  Users that need the same head
count, key width, value width and ring length form a group and share one page numbering; a group
that keeps every key and a group that keeps a window have pools and page tables of their own,
and a window group's pool holds no more pages than its rings can use.

Beside the pages each slot owns a fixed-size float32 state row per user that asks for one
(`Mixer.state_size()`), zeroed when the slot is acquired.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import diagnostics
from ..csrc.build import page_tokens
from ..parts.base import KVNeed
from .slots import CacheError, CacheFull, SlotBook

PAGE = page_tokens()      # LLB_PAGE of csrc/common.cuh: also the attention kernels' key tile


@dataclass(frozen=True)
class CacheConfig:
    """max_tokens: the most tokens all live sequences hold together, each sequence's count
    rounded up to a whole page.  max_seqs: the most live sequences (default: one per page)."""
    max_tokens: int
    max_seqs: Optional[int] = None


def ring_pages(window: Optional[int]) -> Optional[int]:
    """Pages of a ring that always holds the last `window` keys while one page is being filled:
    ceil((window - 1) / PAGE) + 1."""
    if window is None:
        return None
    return -(-(window - 1) // PAGE) + 1


@dataclass
class KVView:
    """What a mixer sees of the cache in one step: its call's pools and the batch's page table."""
    k: torch.Tensor                 # [pages, kv heads, PAGE, key_dim]
    v: Optional[torch.Tensor]       # [pages, kv heads, PAGE, value_dim]; None when the mixer keeps no values
    page_table: torch.Tensor        # int32 [n_seqs, width]
    ring: int
    writable: bool


class PagedCache:
    def __init__(self, needs: List[Optional[KVNeed]], cache_of: List[Optional[int]], state_sizes: List[int],
                 config: CacheConfig, dtype: torch.dtype, device, allocate: bool = True):
        """needs[u], state_sizes[u]: what user u (a mixer of the run order) asks for; cache_of[u]:
        an earlier user whose keys and values user u reads instead of keeping its own."""
        self.config, self.dtype, self.device = config, dtype, torch.device(device)
        n_pages = max(1, -(-config.max_tokens // PAGE))
        self.n_pages = n_pages
        self.n_slots = min(config.max_seqs or n_pages, n_pages) if config.max_seqs else n_pages
        # ---- groups
        self.group_keys: List[tuple] = []
        self.call_group: List[Optional[int]] = []
        self.call_entry: List[Optional[int]] = []
        self.call_owner: List[Optional[int]] = []
        entries_per_group: List[int] = []
        for c, need in enumerate(needs):
            owner = cache_of[c]
            if owner is not None:
                if not (0 <= owner < c) or needs[owner] is None or cache_of[owner] is not None:
                    raise CacheError(f"call {c} reads the cache of call {owner}, which keeps none of its own")
                if needs[owner].window is not None:
                    raise CacheError(f"call {c} reads the cache of call {owner}, which keeps a window only; "
                                     f"a shared cache has to keep every key")
                if need is not None and (need.num_kv_heads, need.key_dim, need.value_dim) != (
                        needs[owner].num_kv_heads, needs[owner].key_dim, needs[owner].value_dim):
                    raise CacheError(f"call {c} reads the cache of call {owner} but their head shapes differ")
                self.call_group.append(self.call_group[owner])
                self.call_entry.append(self.call_entry[owner])
                self.call_owner.append(owner)
                continue
            self.call_owner.append(None)
            if need is None:
                self.call_group.append(None)
                self.call_entry.append(None)
                continue
            key = (need.num_kv_heads, need.key_dim, need.value_dim, ring_pages(need.window))
            if key not in self.group_keys:
                self.group_keys.append(key)
                entries_per_group.append(0)
            g = self.group_keys.index(key)
            self.call_group.append(g)
            self.call_entry.append(entries_per_group[g])
            entries_per_group[g] += 1
        self.rings = [k[3] for k in self.group_keys]
        # a sequence never holds more pages of a window group than its ring has
        self.group_pages = [n_pages if r is None else min(n_pages, r * self.n_slots) for r in self.rings]
        self.book = SlotBook(self.n_slots, self.group_pages, self.rings, PAGE)
        # ---- storage
        self.k_pools: List[torch.Tensor] = []
        self.v_pools: List[torch.Tensor] = []
        self.state: Dict[int, torch.Tensor] = {}
        self.state_sizes = list(state_sizes)
        self._guards: List[tuple] = []            # (what, raw allocation) of every guarded tensor
        if allocate:
            for g, ((nkvh, dk, dv, _), n_entries, pages) in enumerate(zip(self.group_keys, entries_per_group, self.group_pages)):
                self.k_pools.append(self._zeros(f"keys of group {g}", (n_entries, pages, nkvh, PAGE, dk), dtype))
                self.v_pools.append(self._zeros(f"values of group {g}", (n_entries, pages, nkvh, PAGE, dv), dtype)
                                    if dv > 0 else None)
            for c, n in enumerate(state_sizes):
                if n > 0:
                    self.state[c] = self._zeros(f"state of user {c}", (self.n_slots, n), torch.float32)
        diagnostics.log.info("cache: %d pages of %d tokens, %d slots, groups %s, %.1f MB", n_pages, PAGE, self.n_slots,
                             [(k, p) for k, p in zip(self.group_keys, self.group_pages)],
                             sum(p.numel() * p.element_size() for p in self.k_pools + self.v_pools if p is not None) / 1e6)

    def _zeros(self, what: str, shape, dtype) -> torch.Tensor:
        if not diagnostics.CANARY:
            return torch.zeros(shape, dtype=dtype, device=self.device)
        t, raw = diagnostics.guarded(shape, dtype, self.device)
        self._guards.append((what, raw))
        return t

    def check_guards(self) -> None:
        """Raises CacheError naming every guarded tensor whose guard words were overwritten (LLAISYS_CANARY=1)."""
        broken = [what for what, raw in self._guards if not diagnostics.guards_intact(raw)]
        if broken:
            raise CacheError("guard words overwritten around: " + ", ".join(broken))

    # ---- sequences
    def acquire(self) -> int:
        slot = self.book.acquire()
        for st in self.state.values():
            st[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        self.book.release(slot)

    def length(self, slot: int) -> int:
        return self.book.length(slot)

    @property
    def live_slots(self) -> List[int]:
        return sorted(self.book.seqs)

    def bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(p.shape[0] * p.shape[2] * p.shape[4] * es for p in self.k_pools + self.v_pools if p is not None)

    # ---- per-step tables
    def table_width(self, group: int, slots: List[int]) -> int:
        return max(1, max(len(self.book.pages(s, group)) for s in slots))

    def page_table(self, group: int, slots: List[int], width: Optional[int] = None) -> np.ndarray:
        """int32 [len(slots), width]: entry i of a row is the physical page at ring position i."""
        width = width or self.table_width(group, slots)
        t = np.zeros((len(slots), width), dtype=np.int32)
        for r, s in enumerate(slots):
            pages = self.book.pages(s, group)
            t[r, :len(pages)] = pages
        return t

    def ring_of(self, group: int, width: int) -> int:
        """The modulus the kernels use: the ring length, or (no ring) anything >= the width."""
        ring = self.rings[group]
        return ring if ring is not None else max(width, 1)

    def view(self, call: int, tables: Dict[int, torch.Tensor]) -> KVView:
        g = self.call_group[call]
        if g is None:
            raise CacheError(f"call {call} keeps no keys and values")
        table = tables[g]
        e = self.call_entry[call]
        v = self.v_pools[g]
        return KVView(self.k_pools[g][e], v[e] if v is not None else None, table, self.ring_of(g, table.shape[1]),
                      writable=self.call_owner[call] is None)


__all__ = ["PAGE", "CacheConfig", "CacheError", "CacheFull", "KVView", "PagedCache", "ring_pages"]
