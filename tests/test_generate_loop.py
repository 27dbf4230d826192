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


# -- greedy choices that stay on the device: the loop runs one step ahead ---------------------------------------

class AheadEngine(FakeEngine):
    """A FakeEngine whose decode steps choose their tokens themselves, by the Script's rule, and can be run
    again on top of those choices (``step_again``) before the host has read them (``fetch_choices``)."""

    class _Event:
        def synchronize(self):
            pass

    class _Ids(list):
        def tolist(self):
            return list(self)

        def __getitem__(self, k):
            got = list.__getitem__(self, k)
            return AheadEngine._Ids(got) if isinstance(k, slice) else got

    def __init__(self, special=None, **kw):
        super().__init__(**kw)
        self.special, self.owner, self.n_alloc, self.last, self.again = special or {}, {}, 0, None, 0

    def alloc_slot(self):
        s = super().alloc_slot()
        self.owner[s] = self.n_alloc           # requests take their slots in request order
        self.n_alloc += 1
        return s

    def step(self, slots, tokens):
        out = super().step(slots, tokens)
        decode = all(len(t) == 1 for t in tokens)
        self.last = (list(slots), [self.special.get((self.owner[s], n), 100 + n) for s, n in out]) if decode else None
        return out

    def choice_buffer(self, n):
        return None if self.last is None else object()

    def fetch_choices(self, n):
        if self.last is None:
            return None
        assert n == len(self.last[0])
        return self._Event(), self._Ids(self.last[1])

    def step_again(self, slots):
        assert self.last is not None and list(slots) == self.last[0], "only the sequences of the last decode step"
        self.again += 1
        return self.step(slots, [[t] for t in self.last[1]])


def run_ahead(prompts, max_tokens=0, stops=(), special=None, engine=None, **kw):
    engine = engine or AheadEngine(special)
    chooser = Script(special)
    chooser.greedy_on_device = True
    res = generate(engine, chooser, prompts, GenerateParams(max_tokens, GREEDY), stops, **kw)
    assert not engine.held, "every slot goes back"
    return res, engine, chooser


def same(a, b):
    return [(r.stop, r.tokens, r.n_generated, r.n_prompt) for r in a] == [(r.stop, r.tokens, r.n_generated, r.n_prompt) for r in b]


def test_running_ahead_changes_no_result():
    cases = [
        dict(prompts=[[1, 2, 3]], max_tokens=4),
        dict(prompts=[[1, 2]], max_tokens=10, stops=[7], special={(0, 4): 7}),
        dict(prompts=[[1, 2]], stops=[102]),
        dict(prompts=[[1] * 5, [1] * 9, [1] * 13], stops=[107, 112], max_tokens=6),
        dict(prompts=[[1] * 5, [1] * 9, [1] * 13], stops=[107, 112, 114]),
        dict(prompts=[[1] * (i + 1) for i in range(7)], max_tokens=3, max_batch=3),
        dict(prompts=[[1] * 3, [2] * 4], max_tokens=1),
        dict(prompts=[[1] * 3, [2] * 4], max_tokens=2),
    ]
    for case in cases:
        plain, _ = run(**case)
        ahead, eng, chooser = run_ahead(**case)
        assert same(plain, ahead), case
        # the chooser is asked for the first token of a batch only: every later token came from the device
        assert all(len(eng.steps[0]) >= len(c) for c in chooser.calls)
    # a context that fills up
    plain, _ = run([[1] * 60], engine=FakeEngine(max_seq_len=64))
    ahead, eng, _ = run_ahead([[1] * 60], engine=AheadEngine(max_seq_len=64))
    assert same(plain, ahead) and ahead[0].stop == StopReason.CONTEXT_FULL


def test_running_ahead_launches_before_it_reads_and_never_past_a_count_limit():
    # 8 tokens: the first from the prompt step, decode steps for tokens 2..8 = 7 steps as without running ahead
    res, eng, chooser = run_ahead([[1, 2, 3]], max_tokens=8)
    assert res[0].n_generated == 8 and eng.steps == [[3]] + [[1]] * 7
    assert len(chooser.calls) == 1                  # the first token only
    assert eng.again == 6                           # decode steps 2..7 were launched on device tokens; step 1 needs the
    #                                                 host's first token, and nothing runs on top of the last counted token
    # a stop token: the step run ahead has already happened, and nobody sees it
    res, eng, _ = run_ahead([[1, 2]], stops=[7], special={(0, 5): 7}, max_tokens=20)
    assert res[0].stop == StopReason.END_OF_TURN and res[0].tokens == [102, 103, 104]
    assert eng.steps == [[2], [1], [1], [1], [1]]   # one step more than the three tokens needed
    # a callback stop is seen one step late as well
    res, eng, _ = run_ahead([[1]], on_token=lambda i, t: t != 103, max_tokens=20)
    assert res[0].stop == StopReason.CALLBACK and res[0].tokens == [101, 102, 103]


def test_running_ahead_when_one_sequence_stops_the_others_keep_their_step():
    # sequence 0 stops on its third token; the step that ran ahead is sequence 1's next step all the same
    special = {(0, 7): 9}
    plain, _ = run([[1] * 5, [1] * 9], stops=[9], special=special, max_tokens=7)
    ahead, eng, _ = run_ahead([[1] * 5, [1] * 9], stops=[9], special=special, max_tokens=7)
    assert same(plain, ahead)
    assert ahead[0].stop == StopReason.END_OF_TURN and ahead[1].stop == StopReason.MAX_TOKENS
    # every decode step of sequence 1 ran exactly once: prompt + 6 steps for 7 tokens
    assert sum(1 for s in eng.steps[1:]) >= 6


# -- a step whose kernel gave up, sequences that end, a sequence that continues on a slot of the caller's ----------

def test_a_step_that_did_not_finish_raises_and_every_slot_goes_back():
    from nncpu_b200.errors import ExtensionError

    class GivingUp(FakeEngine):
        def check_status(self):
            if len(self.steps) == 3:
                raise ExtensionError("a kernel gave up waiting (status 2)")
    eng = GivingUp()
    seen = []
    with pytest.raises(ExtensionError, match="gave up"):
        generate(eng, Script(), [[1, 2], [3]], GenerateParams(8, GREEDY), on_token=lambda i, t: seen.append(t) or True)
    assert not eng.held
    assert len(seen) == 4                     # the tokens of the third step were never handed out

    class GivingUpAhead(AheadEngine):
        def check_status(self):
            if len(self.steps) == 4:
                raise ExtensionError("a kernel gave up waiting (status 2)")
    eng = GivingUpAhead()
    chooser = Script()
    chooser.greedy_on_device = True
    with pytest.raises(ExtensionError):
        generate(eng, chooser, [[1, 2], [3]], GenerateParams(8, GREEDY))
    assert not eng.held


def test_on_finish_is_called_once_per_sequence_when_it_stops():
    done = []
    res, _ = run([[1], [2, 2], [3, 3, 3]], max_tokens=5, stops=(103,), on_finish=done.append)
    # sequence 2 (three prompt tokens) writes 103 as its first token and ends there, before the others
    assert res[2].stop == StopReason.END_OF_TURN and res[2].n_generated == 0 and done == [2, 1, 0]
    flag = iter([False, False, True])
    done = []
    res, _ = run([[1], [2]], cancelled=lambda: next(flag), on_finish=done.append)
    assert all(r.stop == StopReason.CANCELLED for r in res) and sorted(done) == [0, 1]


def test_continuing_on_a_slot_of_the_callers():
    from nncpu_b200.engine.generate import generate_on_slot
    eng = FakeEngine()
    slot = eng.alloc_slot()
    eng.step([slot], [[7, 8, 9]])                       # three tokens are in the cache already
    context = [7, 8, 9, 10, 11]                         # two more wait
    r = generate_on_slot(eng, Script(), slot, context, 3, GenerateParams(3, GREEDY))
    assert eng.steps[1] == [2] and r.n_prompt == 2 and r.n_generated == 3 and r.stop == StopReason.MAX_TOKENS
    assert context == [7, 8, 9, 10, 11] + r.tokens      # the caller's context grew in place
    assert list(eng.held) == [slot] and eng.held[slot] == len(context) - 1   # kept; the last token waits
    with pytest.raises(InvalidArgument, match="nothing to continue"):
        generate_on_slot(eng, Script(), slot, context, len(context), GenerateParams(1, GREEDY))
    with pytest.raises(ContextFull):
        generate_on_slot(eng, Script(), slot, list(range(64)), 3, GenerateParams(1, GREEDY), n_ctx=64)
    # a stop token joins the context (it ends the reply) but not the result
    n = len(context)
    r = generate_on_slot(eng, Script({(0, n + 1): 999}), slot, context, n - 1, GenerateParams(0, GREEDY), (999,))
    assert r.stop == StopReason.END_OF_TURN and r.n_generated == 1 and context[-1] == 999
    eng.free_slot(slot)
