"""The generation loop's decisions, with scripted stand-ins for the engine and the chooser (no GPU)."""
import pytest

from nncpu_b200.cache import PAGE
from nncpu_b200.engine.generate import generate, plan_batches
from nncpu_b200.errors import ContextFull, InvalidArgument
from nncpu_b200.sampling import GenerateParams, SamplerParams, StopReason

GREEDY = SamplerParams.greedy()


class FakeEngine:
    """Keeps slots and lengths; a step returns, per sequence, (slot, length after the step)."""

    def __init__(self, n_slots=8, max_seq_len=64, n_pages=32):
        self.free, self.held, self.max_seq_len, self.n_pages = list(range(n_slots)), {}, max_seq_len, n_pages
        self.steps, self.max_live = [], 0

    def alloc_slot(self):
        s = self.free.pop()
        self.held[s] = 0
        self.max_live = max(self.max_live, len(self.held))
        return s

    def free_slot(self, s):
        assert s in self.held, "slot freed twice"
        del self.held[s]
        self.free.append(s)

    def step(self, slots, tokens):
        assert len(set(slots)) == len(slots) and all(s in self.held for s in slots)
        for s, t in zip(slots, tokens):
            self.held[s] += len(t)
            assert self.held[s] <= self.max_seq_len
        self.steps.append([len(t) for t in tokens])
        return [(s, self.held[s]) for s in slots]


class Script:
    """Chooses token 100 + (number of tokens the sequence holds), except where told otherwise."""

    def __init__(self, special=None):
        self.special, self.calls = special or {}, []

    def choose(self, logits, indices):
        self.calls.append(list(indices))
        return [self.special.get((i, n), 100 + n) for i, (_, n) in zip(indices, logits)]


def run(prompts, max_tokens=0, stops=(), special=None, engine=None, **kw):
    engine = engine or FakeEngine()
    res = generate(engine, Script(special), prompts, GenerateParams(max_tokens, GREEDY), stops, **kw)
    assert not engine.held, "every slot goes back"
    return res, engine


def test_max_tokens_and_last_token_is_not_evaluated():
    res, eng = run([[1, 2, 3]], max_tokens=4)
    r = res[0]
    assert r.stop == StopReason.MAX_TOKENS and r.n_generated == 4 and r.n_prompt == 3
    assert r.tokens == [103, 104, 105, 106]
    assert eng.steps == [[3], [1], [1], [1]]          # 3 decode steps for 4 tokens


def test_stop_token_is_neither_counted_nor_streamed():
    seen = []
    res, _ = run([[1, 2]], max_tokens=10, stops=[7], special={(0, 4): 7},
                 on_token=lambda i, t: seen.append(t) or True)
    assert res[0].stop == StopReason.END_OF_TURN and res[0].tokens == [102, 103] and seen == [102, 103]
    # a stop token as the very first choice
    res, eng = run([[1, 2]], stops=[102])
    assert res[0].n_generated == 0 and res[0].tokens == [] and eng.steps == [[2]]


def test_callback_stops_one_sequence_only():
    res, _ = run([[1], [1, 2, 3]], max_tokens=5, on_token=lambda i, t: not (i == 0 and t == 102))
    assert res[0].stop == StopReason.CALLBACK and res[0].tokens == [101, 102]  # the token was counted and streamed
    assert res[1].stop == StopReason.MAX_TOKENS and res[1].n_generated == 5


def test_context_full():
    res, _ = run([[1] * 60], engine=FakeEngine(max_seq_len=64))
    assert res[0].stop == StopReason.CONTEXT_FULL and res[0].n_generated == 4
    with pytest.raises(ContextFull):                   # the prompt plus one token must fit
        run([[1] * 64], engine=FakeEngine(max_seq_len=64))
    with pytest.raises(InvalidArgument, match="empty"):
        run([[1], []])


def test_order_of_checks_as_in_the_reference():
    # a stop token wins over everything; context-full is seen before max_tokens
    res, _ = run([[1] * 62], max_tokens=2, engine=FakeEngine(max_seq_len=64))
    assert res[0].stop == StopReason.CONTEXT_FULL and res[0].n_generated == 2
    res, _ = run([[1] * 62], max_tokens=2, stops=[163], engine=FakeEngine(max_seq_len=64))
    assert res[0].stop == StopReason.END_OF_TURN and res[0].n_generated == 1


def test_shorter_sequences_leave_the_batch():
    res, eng = run([[1] * 5, [1] * 9, [1] * 13], stops=[107, 112], max_tokens=6)
    assert [r.stop for r in res] == [StopReason.END_OF_TURN, StopReason.END_OF_TURN, StopReason.MAX_TOKENS]
    assert [r.n_generated for r in res] == [2, 3, 6]
    assert eng.steps == [[5, 9, 13], [1, 1, 1], [1, 1, 1], [1, 1], [1], [1]]


def test_batches_follow_one_another_and_reuse_slots():
    eng = FakeEngine(n_slots=3)
    res, _ = run([[1] * (i + 1) for i in range(7)], max_tokens=2, engine=eng, max_batch=3)
    assert len(res) == 7 and all(r.n_generated == 2 for r in res)
    assert [r.n_prompt for r in res] == list(range(1, 8))
    assert eng.max_live == 3
    assert [s for s in eng.steps if len(s) > 1 or s[0] > 1][0] == [1, 2, 3]
    assert [1, 2, 3] in eng.steps and [4, 5, 6] in eng.steps and [7] in eng.steps


def test_cancel_is_seen_between_steps():
    n = {"calls": 0}

    def cancelled():
        n["calls"] += 1
        return n["calls"] > 2
    res, _ = run([[1], [2, 3]], cancelled=cancelled)
    assert all(r.stop == StopReason.CANCELLED for r in res) and [r.n_generated for r in res] == [2, 2]


def test_plan_batches():
    assert plan_batches([10, 10, 10], [5, 5, 5], 2, 100) == [[0, 1], [2]]
    assert plan_batches([PAGE, PAGE, PAGE], [1, 1, 1], 8, 4) == [[0, 1], [2]]   # two pages each
    with pytest.raises(ContextFull, match="request 1"):
        plan_batches([10, PAGE * 5], [1, 1], 8, 4)


def test_engine_failure_gives_every_slot_back():
    class Failing(FakeEngine):
        def step(self, slots, tokens):
            if len(self.steps) == 2:
                raise RuntimeError("boom")
            return super().step(slots, tokens)
    eng = Failing()
    with pytest.raises(RuntimeError):
        generate(eng, Script(), [[1], [2]], GenerateParams(8, GREEDY))
    assert not eng.held
