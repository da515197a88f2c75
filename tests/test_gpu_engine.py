"""The engine against the plain implementation under every way of cutting requests into steps."""
import numpy as np
import pytest
import torch

from helpers import (CONFIGS, Oracle, build_engine, compare, make_folder, random_requests, run_batches,
                     run_chunked, run_mixed, run_tail_by_one, run_whole)

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]

# request lengths: a single token, page edges (63, 64, 65), the window's ring (B: 2 pages, C: 3), some hundreds
LENGTHS = {"A": [5, 9, 2, 64, 150], "B": [1, 7, 13, 20, 65, 200], "C": [3, 70, 71, 129, 300]}


# Query and key projections are scaled up so that attention is not flat and a lost or misplaced
# key shows in the logits.  Under float32 the scores spread over about +-10; under bfloat16 a
# score's own rounding error grows with its size (|s| * 2^-9) and passes through the softmax, so
# the spread is kept near +-3 there, where that stays inside the bound of helpers.tolerance.
GAIN = {torch.float32: 12.0, torch.bfloat16: 5.0}


class Model:
    def __init__(self, name, tmp):
        self.name, self.requests = name, random_requests(CONFIGS[name], LENGTHS[name], seed=ord(name))
        self._tmp, self._made = tmp, {}

    def __iter__(self):           # (name, folder, oracle, requests) of the float32 variant
        return iter((self.name, *self.at(torch.float32), self.requests))

    def at(self, dtype):
        if dtype not in self._made:
            folder = make_folder(self._tmp / f"gain{int(GAIN[dtype])}", CONFIGS[self.name], seed=ord(self.name),
                                 attn_gain=GAIN[dtype])
            self._made[dtype] = (folder, Oracle(folder))
        return self._made[dtype]


@pytest.fixture(scope="module", params=["A", "B", "C"])
def model(request, tmp_path_factory):
    return Model(request.param, tmp_path_factory.mktemp(f"tiny{request.param}"))


def _rooms(requests):
    return sum(-(-len(r) // 64) * 64 for r in requests)


@pytest.mark.parametrize("dtype", DTYPES)
def test_each_request_alone_and_whole(model, dtype):
    name, requests = model.name, model.requests
    folder, oracle = model.at(dtype)
    engine = build_engine(folder, dtype, max_tokens=max(-(-len(r) // 64) * 64 for r in requests))
    worst = compare(run_whole(engine, requests), oracle, requests, dtype, CONFIGS[name], f"{name} whole")
    print(f"{name} {dtype} whole: worst error/tolerance {worst}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_last_tokens_one_by_one(model, dtype):
    name, requests = model.name, model.requests
    folder, oracle = model.at(dtype)
    engine = build_engine(folder, dtype, max_tokens=max(-(-len(r) // 64) * 64 for r in requests))
    worst = compare(run_tail_by_one(engine, requests), oracle, requests, dtype, CONFIGS[name], f"{name} tail-by-one")
    print(f"{name} {dtype} tail: worst error/tolerance {worst}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_with_slot_reuse(model, dtype):
    name, requests = model.name, model.requests
    folder, oracle = model.at(dtype)
    n = len(requests)
    # two batches, one after the other, in a cache that only just holds the larger one: pages and
    # slots of the first batch are used again by the second
    batches = [list(range(0, n, 2)), list(range(1, n, 2))]
    prompt_lens = [max(1, len(r) - (3 + 5 * i)) for i, r in enumerate(requests)]
    room = max(_rooms([requests[r] for r in b]) for b in batches)
    engine = build_engine(folder, dtype, max_tokens=room, max_seqs=len(batches[0]))
    got = run_batches(engine, requests, batches, prompt_lens)
    worst = compare(got, oracle, requests, dtype, CONFIGS[name], f"{name} batches")
    assert not engine.cache.live_slots and all(p.available == engine.cache.n_pages for p in engine.cache.book.pools)
    # and once more in the other order on the same engine, over the pages the first run dirtied
    got = run_batches(engine, requests, batches[::-1], prompt_lens)
    compare(got, oracle, requests, dtype, CONFIGS[name], f"{name} batches again")
    print(f"{name} {dtype} batches: worst error/tolerance {worst}")


# portions a prompt is fed in: page edges (63, 64, 65), a portion that starts inside the window's ring
# after it has wrapped (B: 2 pages, C: 3), a portion longer than the whole ring, a portion of two
CUTS = [[70, 60, 1000], [63, 1, 64, 65, 2, 1000], [2, 200, 1000], [64]]


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_fed_in_several_portions(model, dtype):
    """A multi-token step on a slot that already holds tokens: the step's queries see the cached
    keys (through a ring that may have wrapped) and the step's own."""
    name = model.name
    folder, oracle = model.at(dtype)
    cfg = CONFIGS[name]
    requests = random_requests(cfg, [200, 300, 129, 9], seed=41)
    engine = build_engine(folder, dtype, max_tokens=320)
    for cuts in CUTS:
        compare(run_chunked(engine, requests, cuts), oracle, requests, dtype, cfg, f"{name} portions {cuts}")
    assert not engine.cache.live_slots


@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_that_mix_single_tokens_prompts_and_portions(model, dtype):
    """In one step one sequence decodes a token onto its history, a second brings a fresh prompt, a
    third a further portion of its prompt, and one sits the step out; run twice over the same
    engine so that slots and pages are used again."""
    name = model.name
    folder, oracle = model.at(dtype)
    cfg = CONFIGS[name]
    requests = random_requests(cfg, [120, 100, 210, 33], seed=43)
    plans = [[50, 1, 1, 1, 40, 1, 0, 1],          # prompt, single tokens, a portion onto history, a pause
             [0, 0, 90],                          # joins at the third step with a 90-token prompt
             [70, 60, 0, 40, 1, 1, 30],           # portions with a pause between them
             [1, 1, 1]]                           # single tokens from an empty slot
    engine = build_engine(folder, dtype, max_tokens=sum(-(-len(r) // 64) * 64 for r in requests), max_seqs=4)
    for turn in range(2):
        got = run_mixed(engine, requests, plans)
        compare(got, oracle, requests, dtype, cfg, f"{name} mixed steps, turn {turn}")
        assert not engine.cache.live_slots
        requests, plans = requests[::-1], plans[::-1]


def test_decoding_past_the_cache_room_of_an_all_window_model():
    """A model whose layers all keep a window can grow past max_tokens positions (its rings never run
    out of pages): the rotary table must cover the model's limit, also for steps replayed from a
    captured graph."""
    import tempfile
    from pathlib import Path
    cfg = CONFIGS["C"]
    with tempfile.TemporaryDirectory() as tmp:
        for dtype in DTYPES:
            folder = make_folder(Path(tmp) / str(dtype), cfg, seed=3, attn_gain=GAIN[dtype])
            oracle = Oracle(folder)
            reqs = random_requests(cfg, [330, 20], seed=2)
            engine = build_engine(folder, dtype, max_tokens=192 + 64, max_seqs=2)      # 256 tokens of room, 330 positions
            assert engine.position_limit == cfg["max_position_embeddings"] and engine.use_graphs
            got = run_batches(engine, reqs, [[0, 1]], [5, 3])
            compare(got, oracle, reqs, dtype, cfg, "all-window model beyond the cache room")
            assert engine.graph_replays > 200


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model, dtype):
    """One short prompt, then some hundred tokens one by one (across several pages and, for
    window layers, several turns of the ring), beside a second sequence that ends early."""
    name = model.name
    folder, oracle = model.at(dtype)
    cfg = CONFIGS[name]
    long_req, short_req = random_requests(cfg, [280, 40], seed=99)
    engine = build_engine(folder, dtype, max_tokens=320 + 64)
    got = run_batches(engine, [long_req, short_req], [[0, 1]], [3, 2])
    compare(got, oracle, [long_req, short_req], dtype, cfg, f"{name} long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens(model, dtype):
    """Positions 0, 1, 2 of a sequence, fed one by one from an empty slot."""
    name = model.name
    folder, oracle = model.at(dtype)
    cfg = CONFIGS[name]
    reqs = random_requests(cfg, [4, 3], seed=5)
    engine = build_engine(folder, dtype, max_tokens=128)
    got = run_batches(engine, reqs, [[0, 1]], [1, 1])
    compare(got, oracle, reqs, dtype, cfg, f"{name} first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_captured_decode_steps_equal_uncaptured_ones(model, dtype):
    """Decode steps are replayed from a CUDA graph once their shape has been seen; that must
    change nothing but rounding (the key range is sliced differently)."""
    name = model.name
    folder, oracle = model.at(dtype)
    cfg = CONFIGS[name]
    reqs = random_requests(cfg, [150, 9, 70], seed=17)
    outs = []
    for graphs in (True, False):
        engine = build_engine(folder, dtype, max_tokens=64 * 5, use_graphs=graphs)
        outs.append(run_batches(engine, reqs, [[0, 1, 2]], [20, 2, 5]))
        assert (engine.graph_replays > 100) == graphs
    compare(outs[0], oracle, reqs, dtype, cfg, f"{name} captured")
    bound = 2e-5 if dtype == torch.float32 else None
    for key, row in outs[1].items():
        if bound:
            assert np.abs(row - outs[0][key]).max() < bound, key


def test_padding_and_company_change_nothing(model):
    """float32: a request's logits are the same alone and in a batch, up to rounding."""
    name, folder, oracle, requests = model
    engine = build_engine(folder, torch.float32, max_tokens=_rooms(requests))
    alone = run_whole(engine, requests)
    together = run_batches(engine, requests, [list(range(len(requests)))], [len(r) for r in requests])
    for key, row in alone.items():
        assert np.abs(row - together[key]).max() < 2e-5, key


def test_step_errors_leave_the_cache_alone(model):
    from llaisys_b200.cache import CacheFull
    from llaisys_b200.engine import StepEntry, StepError
    name, folder, _, requests = model
    cfg = CONFIGS[name]
    engine = build_engine(folder, torch.float32, max_tokens=128, max_seqs=2)
    a, b = engine.acquire(), engine.acquire()
    with pytest.raises(CacheFull):
        engine.acquire()
    with pytest.raises(StepError, match="vocabulary"):
        engine.step([StepEntry(a, [cfg["vocab_size"]], [0])])
    with pytest.raises(StepError, match="twice"):
        engine.step([StepEntry(a, [1], [0]), StepEntry(a, [2], [0])])
    with pytest.raises(StepError, match="wanted"):
        engine.step([StepEntry(a, [1], [1])])
    with pytest.raises(StepError, match="at least one"):
        engine.step([StepEntry(a, [], [])])
    with pytest.raises(CacheFull):
        engine.step([StepEntry(a, [1] * 60, []), StepEntry(b, [1] * 70, [])])       # 64 + 128 > 128
    assert engine.length(a) == 0 and engine.length(b) == 0
    assert engine.cache.book.pools[0].available == engine.cache.n_pages            # the failed step kept no page
    assert engine.step([StepEntry(a, [1, 2, 3], [])]) is None and engine.length(a) == 3
    with pytest.raises(StepError, match="positions"):
        engine.step([StepEntry(b, [1] * (cfg["max_position_embeddings"] + 1), [])])
    engine.release(a)
    engine.release(b)
