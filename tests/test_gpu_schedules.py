"""Ways of cutting and batching the work that the other model tests do not run: a step that mixes sequences
which go on by one token with a newcomer's whole prompt; a decode step whose keys are cut into more splits than
a thread-block cluster holds, inside a captured graph; the benchmark's decode loop against generation through the
entry point; sampled generation one step ahead of the host against the same session kept behind it; and a
one-sequence ``eval`` whose logits outlive a ``generate`` on the same session."""
import numpy as np
import pytest
import torch

from gpu_util import DEV, TOL, check
from nncpu_b200 import Engine, GenerateParams, Model, SamplerParams, Session, SessionParams
from nncpu_b200.kernels import ops
from plain_qwen3 import PlainQwen3, argmax_first
from tiny import make_folder

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("schedules")
    return {(name, dtype): make_folder(root / f"{name}_{dtype}", name, seed=40 + ord(name), store_dtype=STORE[dtype])
            for name in "ABEG" for dtype in DTYPES}


def toks(plain, n, seed):
    return np.random.RandomState(seed).randint(0, plain.cfg.vocab, size=n).tolist()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", "BEG")
def test_decoders_and_a_newcomers_prompt_in_one_step(folders, name, dtype):
    """Sequences a and b are under way and bring one token each; c joins the same step with a prompt of 200
    tokens; a step later d joins with 600 while b has left.  Every logit is the plain model's."""
    plain = PlainQwen3(folders[name, dtype])
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 24)
    a, b, c, d = toks(plain, 46, 1), toks(plain, 95, 2), toks(plain, 203, 3), toks(plain, 602, 4)
    want = {k: plain.logits(v) for k, v in zip("abcd", (a, b, c, d))}
    sa, sb = engine.alloc_slot(), engine.alloc_slot()
    engine.step([sa, sb], [a[:40], b[:90]], [[], []])
    got = {k: [] for k in "abcd"}
    for i in range(2):                                     # two ordinary decode steps (graphs)
        out = engine.step([sa, sb], [[a[40 + i]], [b[90 + i]]])
        got["a"].append(out[0:1].clone())
        got["b"].append(out[1:2].clone())
    sc = engine.alloc_slot()
    out = engine.step([sa, sc, sb], [[a[42]], c[:200], [b[92]]], [[0], [0, 64, 199], [0]])
    got["a"].append(out[0:1].clone())
    got["c"].append(out[1:4].clone())
    got["b"].append(out[4:5].clone())
    engine.free_slot(sb)
    sd = engine.alloc_slot()                               # takes b's slot and pages
    out = engine.step([sd, sa, sc], [d[:600], [a[43]], [c[200]]], [[0, 127, 128, 599], [0], [0]])
    got["d"].append(out[0:4].clone())
    got["a"].append(out[4:5].clone())
    got["c"].append(out[5:6].clone())
    out = engine.step([sa, sc, sd], [[a[44]], [c[201]], [d[600]]])       # all go on by one token
    for r, k in enumerate("acd"):
        got[k].append(out[r:r + 1].clone())
    check(torch.cat(got["a"]), want["a"][40:45], TOL[dtype], "a: under way throughout")
    check(torch.cat(got["b"]), want["b"][90:93], TOL[dtype], "b: leaves after the mixed step")
    check(torch.cat(got["c"]), want["c"][[0, 64, 199, 200, 201]], TOL[dtype], "c: joins with 200 tokens")
    check(torch.cat(got["d"]), want["d"][[0, 127, 128, 599, 600]], TOL[dtype], "d: joins with 600 tokens")
    model.rt.check_status()
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", "BEG")
def test_one_sequences_short_prompt_steps_run_as_captured_graphs(folders, name, dtype):
    """A step in which one sequence brings 2 to 256 tokens and wants its last logits is captured for its padded
    size and replayed: the first step of a size (run kernel by kernel, then captured), a replay for another
    sequence of another length in the same size, and a second turn on a sequence that is under way (positions
    that do not start at 0, keys from earlier turns) all give the plain model's logits; the cache's books stay
    right; and a step that wants other places, or runs with graphs off, takes the ordinary way to the same logits."""
    plain = PlainQwen3(folders[name, dtype])
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 40)
    plain_engine = Engine(model, max_tokens=64 * 12, use_graphs=False)
    sizes_seen = set()
    for k, (first, second) in enumerate([(2, 30), (5, 3), (17, 100), (33, 31), (100, 17), (300, 212), (512, 40), (20, 9)]):
        seq = toks(plain, first + second, 11 * k + first)
        want = plain.logits(seq, rows=[first - 1, first + second - 1])
        s = engine.alloc_slot()
        got = [engine.step([s], [seq[:first]]).clone()]              # a fresh sequence
        got.append(engine.step([s], [seq[first:]]).clone())            # its second turn, on top of the first
        check(torch.cat(got), want, TOL[dtype], f"{first} tokens, then {second} more")
        engine.free_slot(s)
        engine.cache.check()
        sizes_seen.update(g for g in engine.graphs.prompts)
        if first == 100:                                               # the ordinary way: other places wanted, or no graphs
            s = engine.alloc_slot()
            some = engine.step([s], [seq[:first]], want=[[0, first - 1]]).clone()
            check(some[1:], want[:1], TOL[dtype], "two places wanted")
            engine.free_slot(s)
            p = plain_engine.alloc_slot()
            check(plain_engine.step([p], [seq[:first]]).clone(), want[:1], TOL[dtype], "graphs off")
            plain_engine.free_slot(p)
    assert sizes_seen == {16, 32, 64, 128, 256}         # 300 and 512 tokens took the ordinary way
    assert all(g.graph is not None for g in engine.graphs.prompts.values())
    model.rt.check_status()


@pytest.mark.parametrize("dtype,n_prompt", [("bfloat16", 3000), ("float32", 700)])
def test_long_context_decode_inside_a_graph(folders, dtype, n_prompt):
    """An engine sized for 8 192 tokens: one sequence's decode step cuts its keys into more splits than merge
    inside a cluster, so the captured graph holds the scratch-and-merge form; 40 tokens after a long prompt."""
    plain = PlainQwen3(folders["G", dtype])
    model = Model.load(folders["G", dtype], dtype=dtype)
    engine = Engine(model, max_tokens=8192, max_seq_len=8192)
    if dtype == "bfloat16":
        spec = model.spec.layers[0].mixer
        assert ops.attention_decode_splits(1, spec.n_kv_heads, engine.max_seq_len, model.rt.sm_count) > \
            ops.DECODE_CLUSTER_MAX_SPLITS
    seq = toks(plain, n_prompt + 40, 7)
    want = plain.logits(seq, rows=range(n_prompt - 1, n_prompt + 40))
    s = engine.alloc_slot()
    got = [engine.step([s], [seq[:n_prompt]]).clone()]
    for t in seq[n_prompt:]:
        got.append(engine.step([s], [[t]]).clone())
    assert engine.graphs.by_size[1].graph is not None       # the steps did run through the captured graph
    check(torch.cat(got), want, TOL[dtype], f"40 tokens after {n_prompt}")
    model.rt.check_status()


@pytest.mark.parametrize("name", "AG")
def test_the_decode_loop_of_the_benchmark_gives_generations_greedy_tokens(folders, name):
    folder = folders[name, "float32"]
    plain = PlainQwen3(folder)
    model = Model.load(folder, dtype="float32")
    prompts = [toks(plain, n, 20 + n) for n in (5, 33, 70)]
    session = Session(model, SessionParams(n_ctx=256, seed=1, max_batch=3))
    res = session.generate(prompts, GenerateParams(24, SamplerParams.greedy()), stop_token_ids=())
    engine = Engine(model, max_tokens=64 * 12)
    slots = [engine.alloc_slot() for _ in prompts]
    first = torch.empty(3, dtype=torch.int32, device=DEV)
    ops.argmax(engine.step(slots, prompts), first)
    rest = engine.decode_run(slots, first, 23)               # 23 steps: the last generated token is never run
    mine = torch.cat([first[None], rest]).T.tolist()
    assert mine == [r.tokens for r in res]
    for p, r in zip(prompts, res):                           # and both are the plain model's greedy tokens
        seq = list(p)
        for t in r.tokens[:6]:
            assert t == argmax_first(plain.logits(seq)[-1])
            seq.append(t)
    model.rt.check_status()


def test_sampled_generation_ahead_of_the_host_and_behind_it_give_the_same_tokens(folders):
    folder = folders["G", "bfloat16"]
    model = Model.load(folder, dtype="bfloat16")
    rs = np.random.RandomState(3)
    prompts = [rs.randint(0, 410, size=n).tolist() for n in (9, 40, 3, 120)]
    params = GenerateParams(30, SamplerParams(temperature=0.9, top_k=40, top_p=0.95, min_p=0.02))
    stops = [int(x) for x in rs.randint(0, 410, size=25)]    # some sequences end early: the batch shrinks
    out = []
    for ahead in (True, False, True):
        session = Session(model, SessionParams(n_ctx=256, seed=123, max_batch=4, run_ahead=ahead))
        res = session.generate(prompts, params, stop_token_ids=stops)
        out.append([(r.tokens, r.stop) for r in res])
        assert session.engine.cache.slots.n_held == 0
    assert out[0] == out[1] == out[2]
    assert any(len(t) == 30 for t, _ in out[0]) and any(len(t) < 30 for t, _ in out[0])
    model.rt.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_evaluated_logits_outlive_a_generate_call(folders, dtype):
    """eval(prompt); eval([t]) runs through the size-1 decode graph, whose buffer a later generate() of one
    sequence writes again: logits() and sample() must still answer for the session's own sequence."""
    folder = folders["B", dtype]
    plain = PlainQwen3(folder)
    session = Session(Model.load(folder, dtype=dtype), SessionParams(n_ctx=128, seed=2, max_batch=1))
    own = toks(plain, 12, 5)
    session.eval(own[:11])
    session.eval(own[11:])
    want = plain.logits(own)[-1]
    session.generate([toks(plain, 20, 6)], GenerateParams(8, SamplerParams.greedy()), stop_token_ids=())
    check(session.logits(), want, TOL[dtype], "own logits after another request's generation")
    if dtype == "float32":
        assert session.sample(SamplerParams.greedy()) == argmax_first(want)
    assert session.n_past() == 12 and session.tokens() == own


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_step_asks_the_allocator_for_nothing(folders, dtype):
    """The engine's arena is sized when the engine is made; 50 steps of every kind (prompts of unequal lengths,
    mixed steps, decode steps and one sequence's short prompts through graphs after their first) then leave the
    allocator's counters alone."""
    plain = PlainQwen3(folders["G", dtype])
    model = Model.load(folders["G", dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 40, max_step_tokens=2000)
    assert engine.arena.capacity > 0
    rs = np.random.RandomState(9)

    def run(n_steps, check_logits):
        slots, seqs = [], []
        for step in range(n_steps):
            kind = step % 5
            if kind == 0:                                  # a batch starts: prompts of unequal lengths
                for s in slots:
                    engine.free_slot(s)
                lens = [int(x) for x in rs.choice([3, 40, 200, 600], size=rs.randint(1, 4))]
                seqs = [toks(plain, n, 1000 + step + i) for i, n in enumerate(lens)]
                slots = [engine.alloc_slot() for _ in seqs]
                out = engine.step(slots, seqs)
            elif kind == 3 and len(slots) < 4:             # a newcomer's prompt beside the others' next tokens
                new = toks(plain, 90, 2000 + step)
                nxt = [[int(rs.randint(0, plain.cfg.vocab))] for _ in slots]
                slots.append(engine.alloc_slot())
                for q, t in zip(seqs, nxt):
                    q.append(t[0])
                seqs.append(list(new))
                out = engine.step(slots, nxt + [new])
            else:                                          # everybody goes on by one token
                nxt = [[int(rs.randint(0, plain.cfg.vocab))] for _ in slots]
                for q, t in zip(seqs, nxt):
                    q.append(t[0])
                out = engine.step(slots, nxt)
            if check_logits and step % 7 == 0:
                check(out[-1:], plain.logits(seqs[-1], rows=[-1]), TOL[dtype], f"step {step}")
        for s in slots:
            engine.free_slot(s)
    run(15, False)                                         # every path has run once,
    for b in (1, 2, 4):                                    # and every graph size is captured
        slots = [engine.alloc_slot() for _ in range(b)]
        engine.step(slots, [[1, 2, 3]] * b)
        engine.step(slots, [[4]] * b)
        for s in slots:
            engine.free_slot(s)
    for n in (3, 40, 200):                                 # ... and every size of one sequence's short prompt step
        s = engine.alloc_slot()
        engine.step([s], [toks(plain, n, n)])
        engine.free_slot(s)
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    capacity = engine.arena.capacity
    run(50, True)
    torch.cuda.synchronize()
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
    assert engine.arena.capacity == capacity and not engine.arena.overflow
    model.rt.check_status()
