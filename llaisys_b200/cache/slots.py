"""Host-side bookkeeping of the cache: which slots and pages are free, which sequence holds which.

Nothing here touches the device, so the rules (no slot or page lost, held twice or freed
twice) are tested on the CPU.
"""
from __future__ import annotations

from typing import Dict, List


class CacheError(RuntimeError):
    """Misuse of the cache: an unknown or already released slot, and the like."""


class CacheFull(CacheError):
    """No free slot, or not enough free pages for the tokens asked for."""


class FreeList:
    """Integers 0..n-1, handed out lowest-first so that freed ones are used again at once."""

    def __init__(self, n: int, what: str):
        self.n, self.what = n, what
        self._free = list(range(n - 1, -1, -1))     # pop() yields the lowest
        self._held = [False] * n

    @property
    def available(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give_back(self, i: int) -> None:
        if not (0 <= i < self.n):
            raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is not held (freed twice?)")
        self._held[i] = False
        self._free.append(i)
        self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]


class Sequence:
    """What one slot holds: its length and, per group, its physical pages in ring order."""
    __slots__ = ("slot", "length", "pages")

    def __init__(self, slot: int, n_groups: int):
        self.slot, self.length = slot, 0
        self.pages: List[List[int]] = [[] for _ in range(n_groups)]


class SlotBook:
    """Slots (one per live sequence) and, per storage group, a pool of pages.

    groups: list of (ring_pages or None).  A group with ring None keeps every key: a sequence of
    n tokens holds ceil(n / page) pages there.  A group with a ring keeps the last pages only:
    a sequence holds min(ceil(n / page), ring) pages, logical page lp sitting at entry lp % ring.
    """

    def __init__(self, n_slots: int, pages_per_group: List[int], rings: List[int | None], page: int):
        assert len(pages_per_group) == len(rings)
        self.page = page
        self.rings = list(rings)
        self.slots = FreeList(n_slots, "slot")
        self.pools = [FreeList(n, f"page of group {g}") for g, n in enumerate(pages_per_group)]
        self.seqs: Dict[int, Sequence] = {}

    # ---- sequences
    def acquire(self) -> int:
        slot = self.slots.take()
        self.seqs[slot] = Sequence(slot, len(self.pools))
        return slot

    def release(self, slot: int) -> None:
        seq = self._seq(slot)
        for g, pages in enumerate(seq.pages):
            for p in pages:
                self.pools[g].give_back(p)
        del self.seqs[slot]
        self.slots.give_back(slot)

    def _seq(self, slot: int) -> Sequence:
        seq = self.seqs.get(slot)
        if seq is None:
            raise CacheError(f"slot {slot} is not held")
        return seq

    def length(self, slot: int) -> int:
        return self._seq(slot).length

    # ---- pages
    def pages_needed(self, group: int, length: int) -> int:
        n = -(-length // self.page)
        ring = self.rings[group]
        return n if ring is None else min(n, ring)

    def reserve(self, slot: int, n_new: int) -> None:
        """Makes room for n_new more tokens in every group, or raises CacheFull and changes nothing."""
        seq = self._seq(slot)
        want = [self.pages_needed(g, seq.length + n_new) - len(seq.pages[g]) for g in range(len(self.pools))]
        for g, w in enumerate(want):
            if w > self.pools[g].available:
                raise CacheFull(f"slot {slot} needs {w} more pages of group {g} for {n_new} tokens at "
                                f"length {seq.length}; {self.pools[g].available} are free")
        for g, w in enumerate(want):
            for _ in range(max(0, w)):
                seq.pages[g].append(self.pools[g].take())

    def commit(self, slot: int, n_new: int) -> None:
        seq = self._seq(slot)
        for g in range(len(self.pools)):
            if len(seq.pages[g]) < self.pages_needed(g, seq.length + n_new):
                raise CacheError(f"slot {slot}: {n_new} tokens committed without reserved pages")
        seq.length += n_new

    def pages(self, slot: int, group: int) -> List[int]:
        return self._seq(slot).pages[group]

    def audit(self) -> List[str]:
        """Everything that is wrong with the books, in words (empty when they are in order): a slot that is
        live but not held or held but not live, a page that two sequences list or that lies outside its pool,
        a listed page that the pool thinks free, a held page that nobody lists, a sequence with fewer pages
        than its length needs or more than its ring has."""
        bad: List[str] = []
        for slot in self.seqs:
            if not self.slots.is_held(slot):
                bad.append(f"slot {slot} is live but not held")
        for slot in range(self.slots.n):
            if self.slots.is_held(slot) and slot not in self.seqs:
                bad.append(f"slot {slot} is held but holds no sequence")
        for g, pool in enumerate(self.pools):
            owner: Dict[int, int] = {}
            for slot, seq in self.seqs.items():
                pages = seq.pages[g]
                if len(pages) < self.pages_needed(g, seq.length):
                    bad.append(f"slot {slot} holds {len(pages)} pages of group {g}, too few for {seq.length} tokens")
                if self.rings[g] is not None and len(pages) > self.rings[g]:
                    bad.append(f"slot {slot} holds {len(pages)} pages of group {g}, more than its ring of {self.rings[g]}")
                for pg in pages:
                    if not (0 <= pg < pool.n):
                        bad.append(f"slot {slot} lists page {pg} of group {g}, outside the pool (0..{pool.n - 1})")
                        continue
                    if pg in owner:
                        bad.append(f"page {pg} of group {g} is listed by slots {owner[pg]} and {slot}")
                    owner[pg] = slot
                    if not pool.is_held(pg):
                        bad.append(f"slot {slot} lists page {pg} of group {g}, which the pool thinks free")
            for pg in range(pool.n):
                if pool.is_held(pg) and pg not in owner:
                    bad.append(f"page {pg} of group {g} is held but no sequence lists it")
        return bad
