import random

import pytest
import torch

from llaisys_b200.cache import CacheConfig, CacheError, CacheFull, FreeList, PagedCache, SlotBook, ring_pages
from llaisys_b200.parts import KVNeed


def test_free_list_rules():
    f = FreeList(3, "slot")
    assert [f.take(), f.take(), f.take()] == [0, 1, 2]
    with pytest.raises(CacheFull):
        f.take()
    f.give_back(1)
    with pytest.raises(CacheError, match="twice"):
        f.give_back(1)
    with pytest.raises(CacheError):
        f.give_back(7)
    assert f.take() == 1 and f.available == 0          # the freed one is used again


def test_ring_pages():
    assert ring_pages(None) is None
    assert [ring_pages(w) for w in (1, 2, 8, 64, 65, 66, 129, 130)] == [1, 2, 2, 2, 2, 3, 3, 4]


def test_pages_grow_with_length_and_rings_stop_growing():
    book = SlotBook(4, [10, 10], [None, 2], page=64)
    s = book.acquire()
    book.reserve(s, 5); book.commit(s, 5)
    assert len(book.pages(s, 0)) == 1 and len(book.pages(s, 1)) == 1
    book.reserve(s, 60); book.commit(s, 60)               # 65 tokens
    assert len(book.pages(s, 0)) == 2 and len(book.pages(s, 1)) == 2
    book.reserve(s, 200); book.commit(s, 200)              # 265 tokens: 5 pages, ring stays 2
    assert len(book.pages(s, 0)) == 5 and len(book.pages(s, 1)) == 2 and book.length(s) == 265
    with pytest.raises(CacheError, match="without reserved"):
        book.commit(s, 100)
    book.release(s)
    assert book.pools[0].available == 10 and book.pools[1].available == 10 and book.slots.available == 4
    with pytest.raises(CacheError):
        book.release(s)
    with pytest.raises(CacheError):
        book.length(s)


def test_full_pool_changes_nothing():
    book = SlotBook(2, [3], [None], page=64)
    a, b = book.acquire(), book.acquire()
    book.reserve(a, 128); book.commit(a, 128)
    with pytest.raises(CacheFull):
        book.reserve(b, 129)
    assert book.pools[0].available == 1 and book.pages(b, 0) == []
    book.reserve(b, 64)
    with pytest.raises(CacheFull):
        book.acquire()


def test_random_use_loses_nothing():
    rnd = random.Random(0)
    book = SlotBook(5, [40, 40], [None, 3], page=64)
    live = {}
    for _ in range(2000):
        if live and rnd.random() < 0.3:
            s = rnd.choice(list(live))
            book.release(s)
            del live[s]
        elif len(live) < 5 and rnd.random() < 0.5:
            live[book.acquire()] = 0
        elif live:
            s = rnd.choice(list(live))
            n = rnd.randint(1, 150)
            try:
                book.reserve(s, n)
                book.commit(s, n)
                live[s] += n
            except CacheFull:
                pass
        held = [p for s in live for p in book.pages(s, 0)]
        assert len(held) == len(set(held)) and len(held) + book.pools[0].available == 40     # none lost, none twice
        ring = [p for s in live for p in book.pages(s, 1)]
        assert len(ring) == len(set(ring)) and len(ring) + book.pools[1].available == 40
        for s, n in live.items():
            assert book.length(s) == n and len(book.pages(s, 0)) == -(-n // 64) and len(book.pages(s, 1)) == min(3, -(-n // 64))
        assert len(live) + book.slots.available == 5


def _cache(needs, cache_of=None, state=None, max_tokens=640, **kw):
    n = len(needs)
    return PagedCache(needs, cache_of or [None] * n, state or [0] * n, CacheConfig(max_tokens=max_tokens, **kw),
                      torch.float32, "cpu")


def test_groups_have_storage_of_their_own():
    full, win = KVNeed(2, 16, 16, None), KVNeed(2, 16, 16, 8)
    c = _cache([full, win, win, full, KVNeed(1, 32, 32, None), None], state=[0, 0, 0, 0, 0, 12])
    assert c.group_keys == [(2, 16, 16, None), (2, 16, 16, 2), (1, 32, 32, None)]
    assert c.call_group == [0, 1, 1, 0, 2, None] and c.call_entry == [0, 0, 1, 1, 0, None]
    assert c.k_pools[0].shape == (2, 10, 2, 64, 16) and c.k_pools[2].shape == (1, 10, 1, 64, 32)
    assert c.state[5].shape == (10, 12)
    assert c.bytes_per_token() == 2 * 4 * (2 * 2 * 16 + 2 * 2 * 16 + 1 * 32)


def test_keys_and_values_of_different_widths_and_a_mixer_without_values():
    c = _cache([KVNeed(2, 24, 8, None), KVNeed(1, 40, 0, None), KVNeed(2, 24, 8, None)])
    assert c.group_keys == [(2, 24, 8, None), (1, 40, 0, None)] and c.call_entry == [0, 0, 1]
    assert c.k_pools[0].shape == (2, 10, 2, 64, 24) and c.v_pools[0].shape == (2, 10, 2, 64, 8)
    assert c.k_pools[1].shape == (1, 10, 1, 64, 40) and c.v_pools[1] is None
    assert c.bytes_per_token() == 4 * (2 * 2 * (24 + 8) + 40)
    s = c.acquire()
    c.book.reserve(s, 3); c.book.commit(s, 3)
    tables = {g: torch.from_numpy(c.page_table(g, [s])) for g in range(2)}
    v0, v1 = c.view(0, tables), c.view(1, tables)
    assert v0.k.shape == (10, 2, 64, 24) and v0.v.shape == (10, 2, 64, 8) and v1.v is None and v1.writable


def test_a_window_group_holds_no_more_pages_than_its_rings_use():
    c = _cache([KVNeed(1, 8, 8, None), KVNeed(1, 8, 8, 70)], max_tokens=64 * 40, max_seqs=4)
    assert c.rings == [None, 3] and c.group_pages == [40, 12]
    assert c.k_pools[0].shape[1] == 40 and c.k_pools[1].shape[1] == 12
    slots = [c.acquire() for _ in range(4)]
    for s in slots:                                  # every slot can fill its ring, whatever the others hold
        c.book.reserve(s, 600); c.book.commit(s, 600)
    assert c.book.pools[1].available == 0 and all(len(c.book.pages(s, 1)) == 3 for s in slots)


def test_shared_cache_and_state_reset():
    need = KVNeed(2, 16, 16, None)
    c = _cache([need, need, None], cache_of=[None, 0, None], state=[0, 0, 4], max_seqs=3)
    assert c.call_group == [0, 0, None] and c.call_entry == [0, 0, None] and c.call_owner == [None, 0, None]
    assert c.k_pools[0].shape[0] == 1 and c.n_slots == 3
    s = c.acquire()
    c.state[2][s] = 5.0
    c.release(s)
    assert c.acquire() == s and float(c.state[2][s].abs().sum()) == 0.0      # a slot used again starts from zero state
    with pytest.raises(CacheError):
        _cache([need, need], cache_of=[1, None])
    with pytest.raises(CacheError):
        _cache([need, KVNeed(1, 16, 16, None)], cache_of=[None, 0])


def test_page_tables():
    c = _cache([KVNeed(1, 8, 8, None), KVNeed(1, 8, 8, 8)], max_tokens=64 * 8)
    a, b = c.acquire(), c.acquire()
    for s, n in ((a, 200), (b, 3)):
        c.book.reserve(s, n); c.book.commit(s, n)
    t = c.page_table(0, [a, b])
    assert t.shape == (2, 4) and list(t[0]) == c.book.pages(a, 0) and t[1, 0] == c.book.pages(b, 0)[0]
    assert c.page_table(1, [b, a]).shape == (2, 2)
    assert c.ring_of(0, 4) == 4 and c.ring_of(1, 2) == 2
