"""Generation through the Python entry point and the command line against the
plain implementation: greedy, temperature with the reference's chain, stop
tokens, unequal prompts, more requests than the batch holds."""
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT
from nncpu_b200 import (ContextFull, GenerateParams, InvalidArgument, Model, SamplerParams, Session, SessionParams,
                        StopReason)
from plain_qwen3 import PlainMt19937_64, PlainQwen3, argmax_first, sample_chain
from tiny import make_folder

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen")
    out = {}
    for name in "AB":
        folder = make_folder(root / name, name, seed=11)
        out[name] = (folder, PlainQwen3(folder))
    return out


def plain_greedy(plain, prompt, n, stops=()):
    toks, out = list(prompt), []
    for _ in range(n):
        t = argmax_first(plain.logits(toks)[-1])
        if t in stops:
            break
        out.append(t)
        toks.append(t)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_batch_of_unequal_prompts(setup, dtype):
    # the benchmark description's tiny workload: prompts of 5, 9 and 13 tokens, 8 greedy steps
    folder, plain = setup["A"]
    rs = np.random.RandomState(0)
    prompts = [rs.randint(0, 255, size=n).tolist() for n in (5, 9, 13)]
    session = Session(Model.load(folder, dtype=dtype), SessionParams(n_ctx=128, seed=1, max_batch=3))
    res = session.generate(prompts, GenerateParams(8, SamplerParams.greedy()), stop_token_ids=())
    if dtype == "float32":
        for p, r in zip(prompts, res):
            assert r.tokens == plain_greedy(plain, p, 8) and r.stop == StopReason.MAX_TOKENS
            assert (r.n_prompt, r.n_generated) == (len(p), 8) and r.prefill > 0 and r.decode > 0
    else:   # rounding may flip a near-tie; the first tokens still agree
        assert sum(r.tokens[:2] == plain_greedy(plain, p, 2) for p, r in zip(prompts, res)) >= 2
    session.engine.cache.check()
    assert session.engine.cache.slots.n_held == 0


def test_more_requests_than_the_batch_holds_and_stop_tokens(setup):
    folder, plain = setup["B"]
    rs = np.random.RandomState(1)
    prompts = [rs.randint(0, 380, size=n).tolist() for n in (1, 7, 17, 30, 4, 66, 2)]
    session = Session(Model.load(folder, dtype="float32"), SessionParams(n_ctx=128, seed=1, max_batch=3))
    free = [plain_greedy(plain, p, 12) for p in prompts]
    stops = {free[0][3], free[3][0], free[5][11]}
    pieces = []
    res = session.generate(prompts, GenerateParams(12, SamplerParams.greedy()), stop_token_ids=sorted(stops),
                           on_piece=lambda p: pieces.append((p.index, p.token)) or True)
    for i, (p, r) in enumerate(zip(prompts, res)):
        want = plain_greedy(plain, p, 12, stops)
        assert r.tokens == want, i
        assert r.stop == (StopReason.MAX_TOKENS if len(want) == 12 else StopReason.END_OF_TURN)
        assert [t for j, t in pieces if j == i] == want          # streamed in order, stop tokens never
    assert session.engine.cache.slots.n_held == 0
    # the configuration's own end-of-sequence ids are the default
    cfg_stops = session.model.spec.stop_token_ids
    assert cfg_stops == (382, 383)


def test_temperature_with_the_reference_chain(setup):
    # tiny model B, prompts 1/7/17/30, 12 steps at temperature 0.8 with a seeded generator
    folder, plain = setup["B"]
    rs = np.random.RandomState(2)
    prompts = [rs.randint(0, 380, size=n).tolist() for n in (1, 7, 17, 30)]
    params = SamplerParams(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05)
    session = Session(Model.load(folder, dtype="float32"), SessionParams(n_ctx=256, seed=77, max_batch=4))
    res = session.generate(prompts, GenerateParams(12, params), stop_token_ids=())
    for i, (p, r) in enumerate(zip(prompts, res)):
        rng = PlainMt19937_64(77 + i)          # sequence i draws from seed + i on the first generate call
        toks = list(p)
        for t in r.tokens:
            want = sample_chain(plain.logits(toks)[-1], rng, 0.8, 40, 0.95, 0.05)
            assert t == want
            toks.append(t)
    # the same seed gives the same reply whatever else is in the batch
    alone = Session(Model.load(folder, dtype="float32"), SessionParams(n_ctx=256, seed=77, max_batch=1))
    assert alone.generate(prompts[:1], GenerateParams(12, params), stop_token_ids=())[0].tokens == res[0].tokens


def test_temperature_on_the_device(setup):
    folder, plain = setup["A"]
    params = SamplerParams(temperature=1.3, top_k=0, top_p=1.0, min_p=0.0)
    session = Session(Model.load(folder, dtype="float32"), SessionParams(n_ctx=128, seed=5, max_batch=2))
    prompts = [[1, 2, 3], [9, 8, 7, 6]]
    a = session.generate(prompts, GenerateParams(10, params), stop_token_ids=())
    again = Session(session.model, SessionParams(n_ctx=128, seed=5, max_batch=2))
    b = again.generate(prompts, GenerateParams(10, params), stop_token_ids=())
    assert [r.tokens for r in a] == [r.tokens for r in b]
    # each drawn token is what an id-order walk with the same uniform number gives
    for i, (p, r) in enumerate(zip(prompts, a)):
        rng = PlainMt19937_64(5 + i)
        toks = list(p)
        for t in r.tokens:
            l = plain.logits(toks)[-1].astype(np.float64)
            pr = np.exp((l - l.max()) / np.float32(1.3))
            want = int(np.searchsorted(np.cumsum(pr), rng.uniform(1.0) * pr.sum()))
            assert abs(t - want) <= 1
            toks.append(t)


def test_context_full_and_checks(setup):
    folder, _ = setup["A"]
    session = Session(Model.load(folder, dtype="float32"), SessionParams(n_ctx=16, seed=1, max_batch=2))
    res = session.generate([[1] * 12, [2] * 3], GenerateParams(0, SamplerParams.greedy()), stop_token_ids=())
    assert res[0].stop == StopReason.CONTEXT_FULL and res[0].n_generated == 4
    assert res[1].stop == StopReason.CONTEXT_FULL and res[1].n_generated == 13
    with pytest.raises(ContextFull):
        session.generate([[1] * 16])
    with pytest.raises(InvalidArgument):
        session.generate([[]])
    with pytest.raises(InvalidArgument):
        session.generate([[1]], GenerateParams(4, SamplerParams(temperature=-1.0)))
    with pytest.raises(InvalidArgument):
        session.generate([[300]])
    assert session.engine.cache.slots.n_held == 0


def test_cancel_and_callback(setup):
    folder, _ = setup["A"]
    session = Session(Model.load(folder, dtype="float32"), SessionParams(n_ctx=128, seed=1, max_batch=2))
    handle = session.cancel_handle()
    n = []
    res = session.generate([[1, 2], [3]], GenerateParams(50, SamplerParams.greedy()), stop_token_ids=(),
                           on_piece=lambda p: (n.append(p), handle.cancel() if len(n) == 6 else None, True)[2])
    assert all(r.stop == StopReason.CANCELLED for r in res) and [r.n_generated for r in res] == [3, 3]
    res = session.generate([[1, 2]], GenerateParams(5, SamplerParams.greedy()), stop_token_ids=())
    assert res[0].stop == StopReason.MAX_TOKENS            # every call starts uncancelled


def test_one_sequence_calls(setup):
    folder, plain = setup["A"]
    session = Session(Model.load(folder, dtype="float32"), SessionParams(n_ctx=64, seed=3))
    with pytest.raises(InvalidArgument):
        session.sample()
    toks = [5, 6, 7]
    session.eval(toks)
    for _ in range(4):
        want = plain.logits(toks)[-1]
        assert np.abs(session.logits().cpu().numpy() - want).max() < 1e-4
        t = session.sample(SamplerParams.greedy())
        assert t == argmax_first(want)
        session.eval([t])
        toks.append(t)
    assert session.n_past() == 7
    session.reset()
    assert session.n_past() == 0 and session.engine.cache.slots.n_held == 0


def test_command_line_token_run(setup):
    folder, plain = setup["A"]
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "nncpu-b200"), "--gen", str(folder), "5 6 7 8", "6",
                        "--fp32"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = p.stdout.strip().splitlines()
    assert [int(t) for t in lines[0].split()] == plain_greedy(plain, [5, 6, 7, 8], 6, stops=(255,))
    assert lines[1].startswith("prefill: 4 tokens") and lines[2].startswith("decode:") and lines[3].startswith("stop:")
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "nncpu-b200"), "-m", str(folder), "--tokens", "5 6 7 8",
                        "-n", "6", "--temp", "0", "--fp32", "--perf"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.split()] == plain_greedy(plain, [5, 6, 7, 8], 6, stops=(255,))
    assert "tok/s" in p.stderr


def plain_run(plain, prompt, max_tokens, stops, n_ctx):
    """The generation loop's decisions on one request, with the plain model and greedy choices."""
    toks, out = list(prompt), []
    while True:
        t = argmax_first(plain.logits(toks)[-1])
        toks.append(t)
        if t in stops:
            return out, StopReason.END_OF_TURN
        out.append(t)
        if len(toks) >= n_ctx:
            return out, StopReason.CONTEXT_FULL
        if max_tokens > 0 and len(out) >= max_tokens:
            return out, StopReason.MAX_TOKENS


@pytest.mark.parametrize("seed", range(4))
def test_random_generate_calls_on_one_session(tmp_path, seed):
    """Random configurations, three generate() calls each on one session (slots and pages are reused, batches
    follow one another), stop tokens taken from the continuation itself, count and context limits: tokens and
    stop reasons are the plain greedy loop's, in float32."""
    from test_gpu_random_configs import random_config
    from tiny import make_folder
    rs = np.random.RandomState(5000 + seed)
    folder = make_folder(tmp_path / "m", "A", seed=seed, store_dtype=torch.float32, **random_config(rs))
    plain = PlainQwen3(folder)
    n_ctx = int(rs.choice([64, 128, 200]))
    session = Session(Model.load(folder, dtype="float32"),
                      SessionParams(n_ctx=n_ctx, seed=1, max_batch=int(rs.choice([1, 2, 3, 4]))))
    for call in range(3):
        prompts = [rs.randint(0, plain.cfg.vocab, size=int(rs.choice([1, 2, 5, 17, 40, 60]))).tolist()
                   for _ in range(int(rs.randint(1, 7)))]
        max_tokens = int(rs.choice([0, 1, 2, 5, 12, 30]))
        continuation, _ = plain_run(plain, prompts[0], 12, (), n_ctx)
        stops = sorted(set(continuation[2:4])) if rs.rand() < 0.6 else []
        res = session.generate(prompts, GenerateParams(max_tokens, SamplerParams.greedy()), stop_token_ids=stops)
        for i, (p, r) in enumerate(zip(prompts, res)):
            want, why = plain_run(plain, p, max_tokens, stops, n_ctx)
            assert (r.tokens, r.stop) == (want, why), (seed, call, i)
        session.engine.cache.check()
        assert session.engine.cache.slots.n_held == 0


@pytest.mark.parametrize("seed", range(3))
def test_random_sampled_generate_calls_on_one_session(tmp_path, seed):
    """The same with sampling: the chain runs on the device and generation one step ahead of the host; tokens,
    stop reasons and the numbers each sequence draws are the plain loop's with the plain chain."""
    from test_gpu_random_configs import random_config
    from tiny import make_folder
    rs = np.random.RandomState(9000 + seed)
    folder = make_folder(tmp_path / "m", "A", seed=seed, store_dtype=torch.float32, **random_config(rs))
    plain = PlainQwen3(folder)
    n_ctx, session_seed = int(rs.choice([64, 128, 200])), int(rs.randint(1, 1000))
    session = Session(Model.load(folder, dtype="float32"),
                      SessionParams(n_ctx=n_ctx, seed=session_seed, max_batch=int(rs.choice([1, 2, 3, 4]))))
    for call in range(2):
        prompts = [rs.randint(0, plain.cfg.vocab, size=int(rs.choice([1, 3, 9, 30, 50]))).tolist()
                   for _ in range(int(rs.randint(1, 6)))]
        max_tokens = int(rs.choice([1, 3, 8, 20]))
        sp = SamplerParams(float(rs.choice([0.6, 1.0, 1.5])), int(rs.choice([1, 5, 40])), float(rs.choice([1.0, 0.9])),
                           float(rs.choice([0.0, 0.05])))
        stops = [int(x) for x in rs.randint(0, plain.cfg.vocab, size=plain.cfg.vocab // 6)] if rs.rand() < 0.6 else []
        res = session.generate(prompts, GenerateParams(max_tokens, sp), stop_token_ids=stops)
        for i, (p, r) in enumerate(zip(prompts, res)):
            rng = PlainMt19937_64(session_seed + 1000003 * call + i)   # a generator per call and sequence
            toks, out, why = list(p), [], None
            while why is None:
                t = sample_chain(plain.logits(toks)[-1], rng, sp.temperature, sp.top_k, sp.top_p, sp.min_p)
                toks.append(t)
                if t in stops:
                    why = StopReason.END_OF_TURN
                else:
                    out.append(t)
                    if len(toks) >= n_ctx:
                        why = StopReason.CONTEXT_FULL
                    elif len(out) >= max_tokens:
                        why = StopReason.MAX_TOKENS
            assert (r.tokens, r.stop) == (out, why), (seed, call, i)
        session.engine.cache.check()
