"""The diagnostic switches with the engine on the device: results stay those of the plain model, guard words
and audits notice what they are there for (made on the host: nothing here faults a GPU), the timers name the
kernel classes of a step."""
import pytest
import torch

from helpers import CONFIGS, Oracle, build_engine, compare, make_folder, random_requests, run_batches

from llaisys_b200 import diagnostics
from llaisys_b200.cache.slots import CacheError
from llaisys_b200.engine import StepEntry, StepError

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("diag"), CONFIGS["B"], seed=5, attn_gain=5.0)
    return folder, Oracle(folder), random_requests(CONFIGS["B"], [7, 65, 200, 130], seed=11)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_guards_and_audits_change_nothing_and_stay_silent(tiny, dtype, monkeypatch):
    folder, oracle, requests = tiny
    monkeypatch.setattr(diagnostics, "CANARY", True)
    monkeypatch.setattr(diagnostics, "BOUNDS", True)
    batches = [[0, 2], [1, 3]]
    room = max(sum(-(-len(requests[r]) // 64) * 64 for r in b) for b in batches)
    engine = build_engine(folder, dtype, max_tokens=room, max_seqs=2)
    assert engine.cache._guards
    got = run_batches(engine, requests, batches, [max(1, len(r) - 9) for r in requests])
    got = run_batches(engine, requests, batches[::-1], [max(1, len(r) - 4) for r in requests])    # over used pages
    compare(got, oracle, requests, dtype, CONFIGS["B"], "with guards")
    engine.check()
    assert engine.cache.book.audit() == []


def test_an_overwritten_guard_is_reported(tiny, monkeypatch):
    folder, _, requests = tiny
    monkeypatch.setattr(diagnostics, "CANARY", True)
    engine = build_engine(folder, torch.bfloat16, max_tokens=256)
    slot = engine.acquire()
    engine.step([StepEntry(slot, requests[0], [0])])
    engine.check()
    what, raw = engine.cache._guards[0]
    raw[diagnostics.CANARY_WORDS - 1] = 0          # written from the host side of the test: one word before the pool
    with pytest.raises(CacheError, match="guard words overwritten around: " + what):
        engine.check()
    raw[diagnostics.CANARY_WORDS - 1] = diagnostics.CANARY_WORD
    engine.check()
    engine.release(slot)


def test_books_out_of_order_stop_the_step_before_any_launch(tiny, monkeypatch):
    from llaisys_b200.kernels import ops
    folder, _, requests = tiny
    monkeypatch.setattr(diagnostics, "BOUNDS", True)
    engine = build_engine(folder, torch.float32, max_tokens=512)
    a, b = engine.acquire(), engine.acquire()
    engine.step([StepEntry(a, requests[1], []), StepEntry(b, requests[0], [])])
    book = engine.cache.book
    own = book.seqs[b].pages[0][0]
    book.seqs[b].pages[0][0] = book.seqs[a].pages[0][0]            # two sequences would write one page
    n0 = ops.launch_count()
    with pytest.raises(StepError, match="listed by slots"):
        engine.step([StepEntry(a, [1], [0]), StepEntry(b, [2], [0])])
    assert ops.launch_count() == n0 and book.length(a) == len(requests[1]) and book.length(b) == len(requests[0])
    book.seqs[b].pages[0][0] = own
    assert engine.step([StepEntry(a, [1], [0]), StepEntry(b, [2], [0])]).shape[0] == 2
    engine.check()


def test_timers_name_the_kernel_classes_of_a_step(tiny, monkeypatch):
    folder, _, requests = tiny
    timers = diagnostics.KernelTimers(True)
    monkeypatch.setattr(diagnostics, "timers", timers)
    from llaisys_b200.kernels import ops
    monkeypatch.setattr(ops, "timers", timers)
    engine = build_engine(folder, torch.bfloat16, max_tokens=512)
    assert not engine.use_graphs                                    # nothing to time in a replayed graph
    slot = engine.acquire()
    engine.step([StepEntry(slot, requests[2], [0])])
    for t in (3, 4, 5):
        engine.step([StepEntry(slot, [t], [0])])
    engine.check()
    rep = timers.report()
    layers = CONFIGS["B"]["num_hidden_layers"]
    assert rep["embedding"][0] == 4 and rep["add_rmsnorm"][0] == 4 * (2 * layers + 1)
    assert any(k.startswith("attention_prefill") for k in rep) and any(k.startswith("attention_decode") for k in rep)
    assert all(ms >= 0.0 for _, ms in rep.values()) and sum(ms for _, ms in rep.values()) > 0.0
    assert "kernel class" in diagnostics.KernelTimers(True).table()
