"""The generator, the sampling chain and parameter checks (no GPU)."""
import numpy as np
import pytest

from nncpu_b200.errors import InvalidArgument
from nncpu_b200.sampling import Mt19937_64, SamplerParams, argmax_first, sample_from_candidates, sample_from_logits
from plain_qwen3 import PlainMt19937_64, sample_chain


def test_generator_known_answers():
    # values captured from MSVC's std::mt19937_64 (crates/nncpu/src/session/sample.rs:209-224)
    r = Mt19937_64(12345)
    assert [r.next_u64() for _ in range(3)] == [6597103971274460346, 7386862472818278521, 12716877617435052285]
    r = Mt19937_64(42)
    assert [r.uniform(3.5) for _ in range(4)] == [2.643044365340886, 2.236609878491441, 2.632508202618093,
                                                  0.4769543927135297]
    a, b = Mt19937_64(9), PlainMt19937_64(9)
    assert [a.next_u64() for _ in range(700)] == [b.next_u64() for _ in range(700)]


def test_truncation_rules():
    # crates/nncpu/src/session/sample.rs:226-263
    logits = np.array([1.0, 5.0, 3.0, 5.0, -2.0], dtype=np.float32)
    rng = Mt19937_64(1)
    for _ in range(10):
        assert sample_from_logits(logits, SamplerParams(1.0, 1, 1.0, 0.0), rng) == 1   # ties: the lower id
    for _ in range(50):
        assert sample_from_logits(logits, SamplerParams(1.0, 0, 1.0, 0.5), rng) in (1, 3)
    logits = np.array([1.0, 2.0, 7.0, 3.0], dtype=np.float32)
    for _ in range(10):
        assert sample_from_logits(logits, SamplerParams(1e-3, 0, 1.0, 0.0), rng) == 2
    # top_p keeps the smallest prefix that reaches it
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    drawn = {sample_from_logits(logits, SamplerParams(1.0, 0, 0.7, 0.0), rng) for _ in range(200)}
    assert drawn == {0, 1}


def test_nan_is_never_drawn():
    # crates/nncpu/src/session/sample.rs:267-286
    logits = np.full(64, np.nan, dtype=np.float32)
    logits[5], logits[9] = 1.0, 0.5
    rng = Mt19937_64(3)
    for top_k in (0, 2, 40):
        for _ in range(50):
            assert sample_from_logits(logits, SamplerParams(1.0, top_k, 1.0, 0.0), rng) in (5, 9)
    assert argmax_first(logits) == 5
    assert argmax_first(np.array([2.0, 7.0, 7.0], dtype=np.float32)) == 1


def test_chain_matches_the_plain_one():
    rs = np.random.RandomState(0)
    for trial in range(300):
        logits = (rs.randn(60) * 3).astype(np.float32)
        if trial % 5 == 0:
            logits[rs.randint(60)] = np.nan
        if trial % 7 == 0:
            logits[rs.randint(60)] = logits[rs.randint(60)]
        p = SamplerParams(float(rs.choice([0.3, 0.8, 1.0, 1.7])), int(rs.choice([0, 1, 5, 40, 100])),
                          float(rs.choice([1.0, 0.95, 0.5])), float(rs.choice([0.0, 0.05, 0.4])))
        got = sample_from_logits(logits, p, Mt19937_64(trial + 1))
        want = sample_chain(logits, PlainMt19937_64(trial + 1), p.temperature, p.top_k, p.top_p, p.min_p)
        assert got == want, (trial, p)


def test_candidates_of_a_longer_row():
    """The best few of a row, with the row's denominator, give the whole row's draw whenever top-p or
    min-p cuts among them, and say so when neither does."""
    rs = np.random.RandomState(5)
    inside = outside = 0
    for trial in range(200):
        scale = float(rs.choice([0.2, 1.0, 4.0]))
        logits = (rs.randn(500) * scale).astype(np.float32)
        if trial % 6 == 0:
            logits[rs.randint(500, size=9)] = np.nan
        p = SamplerParams(float(rs.choice([0.5, 1.0, 1.4])), 0, float(rs.choice([1.0, 0.9, 0.3])),
                          float(rs.choice([0.0, 0.02, 0.3])))
        if not p.truncates(500):
            continue
        l = np.where(np.isnan(logits), -np.inf, logits).astype(np.float32)
        best = np.lexsort((np.arange(500), -l))[:32]
        total = float(np.exp((l - l.max()).astype(np.float32)).astype(np.float64).sum())
        shuffle = rs.permutation(32)
        got = sample_from_candidates(l[best][shuffle], best[shuffle], p, Mt19937_64(trial + 1), whole_total=total)
        want = sample_chain(logits, PlainMt19937_64(trial + 1), p.temperature, 0, p.top_p, p.min_p)
        if got is None:
            outside += 1
        else:
            inside += 1
            assert got == want, (trial, p)
    assert inside > 50 and outside > 10


def test_distribution_at_temperature():
    logits = np.log(np.array([0.6, 0.3, 0.1], dtype=np.float32))
    rng = Mt19937_64(11)
    n = 4000
    counts = np.bincount([sample_from_logits(logits, SamplerParams(1.0, 0, 1.0, 0.0), rng) for _ in range(n)],
                         minlength=3) / n
    assert np.abs(counts - [0.6, 0.3, 0.1]).max() < 0.03


def test_parameter_checks_and_defaults():
    # crates/nncpu/src/session/mod.rs:101-131
    d = SamplerParams()
    assert (d.temperature, d.top_k, d.top_p, d.min_p) == (0.7, 40, 0.95, 0.05)
    assert SamplerParams.greedy().is_greedy and SamplerParams.greedy().top_k == 40
    for bad in (SamplerParams(-0.1), SamplerParams(float("nan")), SamplerParams(1.0, 0, 1.5, 0.0),
                SamplerParams(1.0, 0, 1.0, -0.1), SamplerParams(1.0, -1), SamplerParams(float("inf"))):
        with pytest.raises(InvalidArgument):
            bad.check()
    assert not SamplerParams(1.0, 0, 1.0, 0.0).truncates(100)
    assert SamplerParams(1.0, 40, 1.0, 0.0).truncates(100) and not SamplerParams(1.0, 100, 1.0, 0.0).truncates(100)
