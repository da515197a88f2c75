"""The switches of llaisys_b200/diagnostics.py: logging, guard words, the audit of the cache's books."""
import logging

import pytest
import torch

from llaisys_b200 import diagnostics
from llaisys_b200.cache.kv import CacheConfig, PagedCache
from llaisys_b200.cache.slots import CacheError, SlotBook
from llaisys_b200.parts.base import KVNeed


def test_logging_is_quiet_by_default_and_speaks_when_asked(capsys):
    log = diagnostics.log
    old_level, old_handlers = log.level, list(log.handlers)
    try:
        log.handlers, log.level = [], logging.NOTSET
        diagnostics.setup_logging("")
        assert not log.handlers
        diagnostics.setup_logging("info")
        diagnostics.setup_logging("info")                    # a second call adds no second handler
        assert len(log.handlers) == 1 and log.level == logging.INFO
        log.info("cache: %d pages", 7)
        log.debug("not shown")
        err = capsys.readouterr().err
        assert "cache: 7 pages" in err and "not shown" not in err
        with pytest.raises(ValueError):
            diagnostics.setup_logging("loud")
    finally:
        log.handlers, log.level = old_handlers, old_level


def test_guard_words_notice_a_write_before_and_after():
    t, raw = diagnostics.guarded((3, 5, 7), torch.bfloat16, "cpu")
    assert t.shape == (3, 5, 7) and t.dtype == torch.bfloat16 and float(t.abs().sum()) == 0.0
    assert t.data_ptr() == raw.data_ptr() + 4 * diagnostics.CANARY_WORDS
    t.fill_(1.5)                                             # the whole body: the guards stay
    assert diagnostics.guards_intact(raw)
    raw[diagnostics.CANARY_WORDS - 1] = 0                    # the word just before the body
    assert not diagnostics.guards_intact(raw)
    t2, raw2 = diagnostics.guarded((10,), torch.float32, "cpu")
    raw2[diagnostics.CANARY_WORDS + 10] = 123                # the word just behind it
    assert not diagnostics.guards_intact(raw2)


def test_the_cache_under_guard(monkeypatch):
    monkeypatch.setattr(diagnostics, "CANARY", True)
    needs = [KVNeed(2, 8, 8, None), KVNeed(2, 8, 4, 70)]
    cache = PagedCache(needs, [None, None], [0, 6], CacheConfig(max_tokens=512, max_seqs=3), torch.float32, "cpu")
    assert len(cache._guards) == 5                           # two key pools, two value pools, one state table
    cache.check_guards()
    s = cache.acquire()
    cache.k_pools[0].fill_(1.0); cache.v_pools[1].fill_(2.0); cache.state[1].fill_(3.0)
    cache.check_guards()
    what, raw = cache._guards[1]
    raw[-1] = 0
    with pytest.raises(CacheError, match="values of group 0"):
        cache.check_guards()
    cache.release(s)


def test_without_the_switch_nothing_is_guarded():
    assert diagnostics.CANARY is False
    cache = PagedCache([KVNeed(1, 8, 8, None)], [None], [0], CacheConfig(max_tokens=128), torch.float32, "cpu")
    assert cache._guards == []
    cache.check_guards()


def test_audit_of_the_books():
    book = SlotBook(3, [8, 4], [None, 2], 64)
    a, b = book.acquire(), book.acquire()
    book.reserve(a, 130); book.commit(a, 130)
    book.reserve(b, 70); book.commit(b, 70)
    assert book.audit() == []
    # a page listed twice
    stolen = book.seqs[a].pages[0][0]
    keep = book.seqs[b].pages[0][0]
    book.seqs[b].pages[0][0] = stolen
    msgs = book.audit()
    assert any("listed by slots" in m for m in msgs) and any(f"page {keep} of group 0 is held but no sequence" in m for m in msgs)
    book.seqs[b].pages[0][0] = keep
    assert book.audit() == []
    # a page outside the pool, a length without pages, a page the pool thinks free
    book.seqs[b].pages[1].append(99)
    assert any("outside the pool" in m for m in book.audit()) and any("more than its ring" in m for m in book.audit())
    book.seqs[b].pages[1].pop()
    book.seqs[a].length = 1000
    assert any("too few" in m for m in book.audit())
    book.seqs[a].length = 130
    book.pools[0]._held[book.seqs[a].pages[0][1]] = False
    assert any("thinks free" in m for m in book.audit())
    book.pools[0]._held[book.seqs[a].pages[0][1]] = True
    # a slot that is held but holds nothing
    book.slots._held[2] = True
    assert any("holds no sequence" in m for m in book.audit())
    book.slots._held[2] = False
    assert book.audit() == []
    book.release(a); book.release(b)
    assert book.audit() == []


def test_timers_cost_nothing_when_off():
    t = diagnostics.KernelTimers(False)
    t.start(); t.mark("linear")
    assert t.report() == {} and t._marks == []
