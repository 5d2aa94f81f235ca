"""The generation loop's decisions, with a scripted engine in place of the GPU:
batches cut to the cache, stop tokens, rows that end early, slots given back,
one batch after another."""
import pytest

from zlm_b200.engine.generate import BatchDecisions, _Row, generate, plan_batches
from zlm_b200.sampling import SamplingParams, uniform_for


class ScriptedEngine:
    """Emits, for request r, the tokens script[r] one after another; counts slots."""

    class Cfg:
        eos_token_ids = (99,)

    def __init__(self, script, max_tokens=64 * 8, max_batch=3, max_seq_len=256):
        self.config = self.Cfg()
        self.script = script
        self.max_tokens, self.max_batch, self.max_seq_len = max_tokens, max_batch, max_seq_len
        self.free = list(range(max_batch))
        self.held = {}
        self.cursor = {}
        self.log = []
        self.max_live = 0

    def new_sequence(self):
        s = self.free.pop(0)
        self.held[s] = 0
        self.max_live = max(self.max_live, len(self.held))
        return s

    def release(self, slot):
        assert slot in self.held, f"slot {slot} freed twice"
        del self.held[slot]
        self.free.append(slot)
        self.free.sort()

    def _next(self, req):
        i = self.cursor.get(req, 0)
        self.cursor[req] = i + 1
        return self.script[req][i]

    def prefill_sample(self, slots, prompts, params, requests):
        self.log.append(("prefill", list(requests), [len(p) for p in prompts]))
        for s, p in zip(slots, prompts):
            assert self.held[s] == 0
            self.held[s] = len(p)
        return [self._next(r) for r in requests]

    def decode_sample(self, slots, tokens, params, requests):
        self.log.append(("decode", list(requests), list(tokens)))
        for s in slots:
            self.held[s] += 1
            assert self.held[s] <= self.max_seq_len
        return [self._next(r) for r in requests]


def test_plan_batches_respects_cache_and_batch_size():
    # 8 pages: 100+29 -> 3 pages, 10+29 -> 1, 200+29 -> 4, 64+29 -> 2
    assert plan_batches([100, 10, 200, 64], 30, 64 * 8, 3, 1024) == [[0, 1, 2], [3]]
    assert plan_batches([100, 10, 200, 64], 30, 64 * 8, 2, 1024) == [[0, 1], [2, 3]]
    assert plan_batches([10] * 5, 1, 64 * 2, 8, 1024) == [[0, 1], [2, 3], [4]]
    with pytest.raises(ValueError, match="empty prompt"):
        plan_batches([3, 0], 4, 640, 2, 100)
    with pytest.raises(ValueError, match="exceeds the longest sequence"):
        plan_batches([101], 4, 640, 2, 100)
    with pytest.raises(ValueError, match="do not fit the cache"):
        plan_batches([100], 400, 128, 2, 1000)
    # the longest sequence caps what a request can ever hold
    assert plan_batches([90], 400, 128, 2, 100) == [[0]]


def test_decisions_stop_length_context():
    d = BatchDecisions(max_tokens=3, stop_ids=[99], max_seq_len=12)
    rows = [_Row(0, 0, 5), _Row(1, 1, 5, out=[7, 8]), _Row(2, 2, 12), _Row(3, 3, 5)]
    live, ended = d.apply(rows, [4, 6, 5, 99])
    assert [r.request for r in live] == [0]
    assert {r.request: (r.out, r.reason) for r in ended} == {
        1: ([7, 8, 6], "length"), 2: ([5], "context"), 3: ([], "stop")}
    d2 = BatchDecisions(3, [99], 12, include_stop=True)
    _, e = d2.apply([_Row(0, 0, 5)], [99])
    assert e[0].out == [99]


def test_rows_end_early_and_slots_come_back():
    script = {0: [1, 2, 99], 1: [3, 99], 2: [4, 5, 6, 7, 8, 9], 3: [99], 4: [10, 11, 12, 13]}
    eng = ScriptedEngine(script)
    seen = []
    res = generate(eng, [[1] * 5, [2] * 3, [3] * 9, [4] * 2, [5] * 7], max_tokens=4,
                   on_token=lambda r, t: seen.append((r, t)))
    assert res.tokens == [[1, 2], [3], [4, 5, 6, 7], [], [10, 11, 12, 13]]
    assert res.finish_reasons == ["stop", "stop", "length", "stop", "length"]
    assert eng.held == {} and eng.max_live == 3
    # batch 1 = requests 0..2; its rows leave one by one, the last token is never fed back
    assert eng.log[0] == ("prefill", [0, 1, 2], [5, 3, 9])
    assert eng.log[1] == ("decode", [0, 1, 2], [1, 3, 4])
    assert eng.log[2] == ("decode", [0, 2], [2, 5])
    assert eng.log[3] == ("decode", [2], [6])
    assert eng.log[4] == ("prefill", [3, 4], [2, 7])
    assert eng.log[5:] == [("decode", [4], [10]), ("decode", [4], [11]), ("decode", [4], [12])]
    assert seen == [(0, 1), (1, 3), (2, 4), (0, 2), (2, 5), (2, 6), (2, 7), (4, 10), (4, 11), (4, 12), (4, 13)]
    s = res.stats
    assert (s.batches, s.prefill_steps, s.decode_steps, s.prompt_tokens, s.new_tokens) == (2, 2, 6, 26, 11)


def test_context_limit_and_explicit_stop_ids():
    eng = ScriptedEngine({0: list(range(1, 50))}, max_seq_len=12)
    res = generate(eng, [[7] * 10], max_tokens=40)
    # positions 10 and 11 can still be fed; the token chosen after the cache is full is kept, not fed
    assert res.tokens == [[1, 2, 3]] and res.finish_reasons == ["context"] and eng.held == {}
    eng = ScriptedEngine({0: [5, 6, 99, 7, 8]})
    assert generate(eng, [[1]], max_tokens=4, stop_token_ids=[6]).tokens == [[5]]
    eng = ScriptedEngine({0: [5, 6, 99, 7, 8]})
    assert generate(eng, [[1]], max_tokens=4, stop_token_ids=()).tokens == [[5, 6, 99, 7]]
    assert generate(ScriptedEngine({0: [1]}), [[1]], max_tokens=0).tokens == [[]]


def test_slots_are_released_when_a_step_fails():
    class Failing(ScriptedEngine):
        def decode_sample(self, *a):
            raise RuntimeError("boom")
    eng = Failing({0: [1, 2], 1: [3, 4]})
    with pytest.raises(RuntimeError, match="boom"):
        generate(eng, [[1], [2]], max_tokens=3)
    assert eng.held == {}


def test_sampling_params_and_uniforms():
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1)
    with pytest.raises(ValueError):
        SamplingParams(temperature=1, top_p=-0.1)
    assert SamplingParams().greedy and not SamplingParams(temperature=0.5).greedy
    # the reference's edge cases (src/runtime/sampler.zig:85-110): top_k 1 and top_p 0 are greedy
    # even with a temperature; top_p of 1 or more keeps the whole support
    assert SamplingParams(temperature=1.5, top_k=1).greedy and SamplingParams(temperature=1, top_p=0).greedy
    assert SamplingParams(temperature=1, top_p=3.0).top_p == 1.0 and not SamplingParams(temperature=1, top_p=3.0).greedy
    us = [uniform_for(3, r, p) for r in range(20) for p in range(50)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) > 990
    assert abs(sum(us) / len(us) - 0.5) < 0.03
    assert uniform_for(3, 1, 2) == uniform_for(3, 1, 2) != uniform_for(4, 1, 2)


class QueueingEngine(ScriptedEngine):
    """The scripted engine with steps that can be queued one ahead, as the GPU engine has
    them: a step fed ``None`` takes, for the same rows, the tokens that the step queued
    before it sampled.  A row of such a step that had already met its stop token computes
    something nobody looks at; every row that goes on must have been fed its own token."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.unfetched = 0
        self.last = None                      # (requests, sampled) of the newest queued step
        self.wasted = 0

    def decode_launch(self, slots, tokens, params, requests):
        assert self.unfetched < 2, "more than two steps in flight"
        if tokens is None:
            assert self.last is not None and list(requests) == self.last[0], "a step fed from the device must keep its rows"
            tokens = self.last[1]
        sampled = []
        for s, r, tok in zip(slots, requests, tokens):
            assert s in self.held, "a freed slot was stepped"
            self.held[s] += 1
            assert self.held[s] <= self.max_seq_len
            i = self.cursor.get(r, 0)
            if i > 0 and self.script[r][i - 1] == 99 and 99 in self.stop_ids:
                self.wasted += 1                                   # the row met its stop token one step ago
                sampled.append(-1)
                continue
            assert tok == self.script[r][i - 1], f"request {r} was fed {tok}, its last token is {self.script[r][i - 1]}"
            sampled.append(self._next(r))
        self.log.append(("decode", list(requests), list(tokens)))
        self.last = (list(requests), sampled)
        self.unfetched += 1
        return sampled

    def decode_fetch(self, handle):
        self.unfetched -= 1
        return handle

    def decode_sample(self, *a):
        raise AssertionError("the loop should queue its steps")

    stop_ids = (99,)


@pytest.mark.parametrize("max_tokens", [1, 2, 4, 7])
def test_steps_queued_one_ahead_give_the_same_tokens(max_tokens):
    script = {0: [1, 2, 99, 50, 51, 52, 53, 54], 1: [3, 99, 60, 61, 62, 63, 64, 65], 2: [4, 5, 6, 7, 8, 9, 10, 11],
              3: [99, 70, 71, 72, 73, 74, 75, 76], 4: [10, 11, 12, 13, 14, 15, 16, 17], 5: [20, 21, 22, 23, 24, 99, 25, 26]}
    prompts = [[1] * 5, [2] * 3, [3] * 9, [4] * 2, [5] * 7, [6] * 4]
    plain = ScriptedEngine(script)
    want = generate(plain, prompts, max_tokens=max_tokens)
    seen = []
    eng = QueueingEngine(script)
    got = generate(eng, prompts, max_tokens=max_tokens, on_token=lambda r, t: seen.append((r, t)))
    assert got.tokens == want.tokens and got.finish_reasons == want.finish_reasons
    assert eng.held == {} and eng.unfetched == 0 and eng.max_live == 3
    for r, toks in enumerate(got.tokens):
        assert [t for q, t in seen if q == r] == toks          # every token reported once, in order
    # a row is computed for nothing at most once: in the step queued before its stop token was read
    assert eng.wasted <= sum(reason == "stop" for reason in got.finish_reasons)


def test_queued_steps_respect_the_context_limit_and_failures():
    eng = QueueingEngine({0: list(range(1, 50))}, max_seq_len=12)
    res = generate(eng, [[7] * 10], max_tokens=40)
    assert res.tokens == [[1, 2, 3]] and res.finish_reasons == ["context"] and eng.held == {}

    class Failing(QueueingEngine):
        def decode_launch(self, *a):
            if len(self.log) >= 2:
                raise RuntimeError("boom")
            return super().decode_launch(*a)
    eng = Failing({0: [1, 2, 3, 4], 1: [3, 4, 5, 6]})
    with pytest.raises(RuntimeError, match="boom"):
        generate(eng, [[1], [2]], max_tokens=4)
    assert eng.held == {}
