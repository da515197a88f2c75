"""The generation loop's decisions, with a scripted engine and sampler (no device)."""
import pytest

from llaisys_b200.engine import GenerationLoop


class FakeEngine:
    page = 64

    def __init__(self, max_tokens=64 * 8, max_seqs=4, max_positions=1000):
        self.max_tokens, self.max_seqs, self.max_positions = max_tokens, max_seqs, max_positions
        self.free = list(range(max_seqs))
        self.held = {}                       # slot -> tokens fed so far
        self.log = []                        # per step: [(slot, tokens, want)]
        self.acquired = []

    def acquire(self):
        assert self.free, "acquire with no free slot"
        s = min(self.free)
        self.free.remove(s)
        self.held[s] = []
        self.acquired.append(s)
        return s

    def release(self, s):
        assert s in self.held, f"slot {s} released twice or never acquired"
        del self.held[s]
        self.free.append(s)

    def step(self, entries):
        rec = []
        for e in entries:
            assert e.slot in self.held
            self.held[e.slot] += list(e.tokens)
            assert len(self.held[e.slot]) <= self.max_positions
            rec.append((e.slot, list(e.tokens), list(e.want)))
        used = sum(-(-len(t) // self.page) * self.page for t in self.held.values())
        assert used <= self.max_tokens, "the loop overfilled the cache"
        self.log.append(rec)
        return [e.slot for e in entries]


def scripted(script):
    calls = []

    def sampler(logits, keys, steps):
        calls.append((list(keys), list(steps)))
        return [script[k][s] for k, s in zip(keys, steps)]
    sampler.calls = calls
    return sampler


def test_unequal_prompts_stop_tokens_and_early_ends():
    eng = FakeEngine()
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9]]
    script = {0: [10, 11, 99, 12], 1: [99], 2: [20, 21, 22, 23, 24, 25]}
    loop = GenerationLoop(eng, scripted(script), stop_ids=[99])
    out = loop.run(prompts, max_new_tokens=5)
    assert [g.tokens for g in out] == [[10, 11, 99], [99], [20, 21, 22, 23, 24]]
    assert [g.reason for g in out] == ["stop", "stop", "length"]
    # first step: all prompts whole, logits wanted at each prompt's last token
    assert [(t, w) for _, t, w in eng.log[0]] == [([1, 2, 3], [2]), ([4], [0]), ([5, 6, 7, 8, 9], [4])]
    # request 1 ended after its first token: the second step holds requests 0 and 2 with one token each
    assert [t for _, t, _ in eng.log[1]] == [[10], [20]] and all(w == [0] for _, _, w in eng.log[1])
    assert [len(s) for s in eng.log] == [3, 2, 2, 1, 1]
    assert not eng.held and sorted(eng.free) == [0, 1, 2, 3]
    assert loop.batches_run == 1 and loop.steps_run == 5


def test_batches_follow_one_another_and_slots_are_used_again():
    eng = FakeEngine(max_seqs=2)
    prompts = [[1] * 3, [2] * 5, [3] * 2, [4] * 4, [5]]
    script = {r: [7] * 10 for r in range(5)}
    script[2] = [7, 0]
    loop = GenerationLoop(eng, scripted(script), stop_ids=[0])
    out = loop.run(prompts, max_new_tokens=3)
    assert [len(g.tokens) for g in out] == [3, 3, 2, 3, 3]
    assert loop.batches_run == 3
    assert eng.acquired == [0, 1, 0, 1, 0]           # the same slots again
    assert not eng.held


def test_admission_respects_cache_size_and_max_batch():
    eng = FakeEngine(max_tokens=64 * 3, max_seqs=8)
    prompts = [[1] * 60, [1] * 70, [1] * 10, [1] * 10]       # rooms with 4 new tokens: 64, 128, 64, 64
    loop = GenerationLoop(eng, scripted({r: [5] * 9 for r in range(4)}))
    loop.run(prompts, max_new_tokens=4)
    assert loop.batches_run == 2 and [len(s) for s in eng.log][0] == 2
    eng = FakeEngine()
    loop = GenerationLoop(eng, scripted({r: [5] * 9 for r in range(4)}), max_batch=1)
    loop.run([[1], [2], [3], [4]], max_new_tokens=2)
    assert loop.batches_run == 4
    with pytest.raises(ValueError, match="room"):
        GenerationLoop(FakeEngine(max_tokens=64), scripted({0: [1] * 99})).run([[1] * 100], 4)


def test_position_limit_and_degenerate_requests():
    eng = FakeEngine(max_positions=6)
    out = GenerationLoop(eng, scripted({0: [5] * 9})).run([[1, 2, 3]], max_new_tokens=9)
    assert out[0].tokens == [5, 5, 5] and out[0].reason == "limit"       # positions 3, 4, 5 filled, then full
    with pytest.raises(ValueError, match="empty"):
        GenerationLoop(FakeEngine(), scripted({})).run([[]], 3)
    with pytest.raises(ValueError, match="no position"):
        GenerationLoop(FakeEngine(max_positions=3), scripted({})).run([[1, 2, 3]], 3)
    out = GenerationLoop(FakeEngine(), scripted({})).run([[1, 2]], 0)
    assert out[0].tokens == [] and out[0].reason == "length"


def test_sampler_sees_request_keys_and_draw_counts():
    s = scripted({0: [1, 2, 3], 1: [4, 5, 6]})
    GenerationLoop(FakeEngine(), s).run([[9], [9, 9]], max_new_tokens=3)
    assert s.calls == [([0, 1], [0, 0]), ([0, 1], [1, 1]), ([0, 1], [2, 2])]


def test_slots_are_returned_when_a_step_fails():
    eng = FakeEngine()

    def boom(entries):
        raise RuntimeError("device fell over")
    eng.step = boom
    with pytest.raises(RuntimeError):
        GenerationLoop(eng, scripted({})).run([[1], [2]], 2)
    assert not eng.held
