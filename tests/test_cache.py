"""Slots, pages, windows and per-sequence state (no GPU; the cache's tensors live on the CPU here)."""
import random

import pytest
import torch

from nncpu_b200.cache import PAGE, Cache, IndexPool, KVRequest, StateRequest, pages_for
from nncpu_b200.errors import ContextFull, InvalidArgument


def make(max_tokens=PAGE * 8, window=0, state=False, **kw):
    reqs = [(KVRequest(2, 16, 0), None), (KVRequest(2, 16, window), StateRequest((3,)) if state else None),
            (KVRequest(2, 16, 0), None)]
    return Cache(reqs, [None, None, None], max_tokens, torch.float32, "cpu", **kw)


def test_pool_never_loses_or_doubles():
    p = IndexPool(4, "thing")
    got = [p.take() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and p.n_free == 0
    with pytest.raises(ContextFull):
        p.take()
    p.give_back(2)
    with pytest.raises(InvalidArgument, match="not in use"):
        p.give_back(2)                       # freed twice
    with pytest.raises(InvalidArgument, match="does not exist"):
        p.give_back(7)
    assert p.take() == 2                     # given back last, handed out first
    p.check()


def test_groups_by_need():
    c = make(window=40)
    assert len(c.groups) == 2                # all keys / a window of them: storage of their own
    assert c.group_of(0) == c.group_of(2) != c.group_of(1)
    assert c.groups[c.group_of(0)].k.shape == (2, 8, 2, PAGE, 16)
    assert c.groups[c.group_of(1)].k.shape == (1, 8, 2, PAGE, 16)
    k0, _ = c.kv(0)
    k2, _ = c.kv(2)
    assert k0.data_ptr() != k2.data_ptr() and k0.shape == (8, 2, PAGE, 16)
    assert make(window=0).groups[0].k.shape[0] == 3 and len(make(window=0).groups) == 1


def test_entry_reading_another_entrys_cache():
    reqs = [(KVRequest(1, 16), None), (None, None), (KVRequest(1, 16), None)]
    c = Cache(reqs, [None, 0, None], PAGE * 2, torch.float32, "cpu")
    assert c.owns_kv(0) and not c.owns_kv(1) and c.owns_kv(2)
    assert c.kv(1)[0].data_ptr() == c.kv(0)[0].data_ptr()
    assert c.groups[0].k.shape[0] == 2       # the reader owns no storage
    with pytest.raises(InvalidArgument, match="earlier entry"):
        Cache(reqs, [None, 2, None], PAGE, torch.float32, "cpu")


def test_step_bookkeeping_and_reuse():
    c = make()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.prepare([a, b], [70, 5])
    assert c.block_table(0, [a, b]) == [c.groups[0].tables[a], c.groups[0].tables[b] + [-1]]
    c.commit([a, b], [70, 5])
    assert (c.length(a), c.length(b)) == (70, 5)
    assert c.groups[0].pool.n_held == 3
    for _ in range(60):                      # b crosses a page boundary while decoding
        c.prepare([a, b], [1, 1])
        c.commit([a, b], [1, 1])
    assert c.length(b) == 65 and len(c.groups[0].tables[b]) == 2 and len(c.groups[0].tables[a]) == 3
    c.check()
    pages_of_b = list(c.groups[0].tables[b])
    c.free_slot(b)                           # the shorter request ends earlier
    assert c.groups[0].pool.n_held == 3
    with pytest.raises(InvalidArgument):
        c.free_slot(b)
    with pytest.raises(InvalidArgument):
        c.prepare([b], [1])
    d = c.alloc_slot()                       # the next request reuses slot and pages
    assert d == b and c.length(d) == 0
    c.prepare([d], [100])
    assert set(pages_of_b) <= set(c.groups[0].tables[d])
    c.check()


def test_context_full_changes_nothing():
    c = make(max_tokens=PAGE * 4)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.prepare([a], [PAGE * 3])
    c.commit([a], [PAGE * 3])
    before = (c.groups[0].pool.n_free, dict(c.groups[0].tables))
    with pytest.raises(ContextFull, match="cache pages"):
        c.prepare([b], [PAGE + 1])
    assert (c.groups[0].pool.n_free, dict(c.groups[0].tables)) == before
    c.prepare([b], [PAGE])
    short = make(max_tokens=PAGE * 4, max_seq_len=100)
    s = short.alloc_slot()
    with pytest.raises(ContextFull, match="at most 100"):
        short.prepare([s], [101])
    with pytest.raises(InvalidArgument, match="twice"):
        c.prepare([a, a], [1, 1])
    with pytest.raises(InvalidArgument):
        c.prepare([a], [0])


def test_window_group_gives_pages_back():
    c = make(max_tokens=PAGE * 8, window=40)
    s = c.alloc_slot()
    full, win = c.groups[c.group_of(0)], c.groups[c.group_of(1)]
    c.prepare([s], [200])
    assert len(win.tables[s]) == pages_for(200)      # the prompt step needs every page
    c.commit([s], [200])
    # a query at position 200 sees keys 161..200: pages 0 and 1 hold nothing it can see
    assert win.tables[s][:2] == [-1, -1] and win.tables[s][2] >= 0
    assert win.pool.n_held == 2 and full.pool.n_held == 4
    for _ in range(120):
        c.prepare([s], [1])
        c.commit([s], [1])
    assert win.first_needed_page(320) == (320 + 1 - 40) // PAGE == 4
    assert [p >= 0 for p in win.tables[s]] == [False] * 4 + [True]
    c.check()
    with pytest.raises(InvalidArgument, match="window"):
        c.truncate(s, 100)
    c.free_slot(s)
    assert win.pool.n_held == 0 and full.pool.n_held == 0
    c.check()


def test_state_is_per_slot_and_cleared_on_start():
    c = make(state=True)
    st = c.state(1)
    assert st.shape == (c.n_slots + 1, 3) and c.state(0) is None   # one spare row for padding
    a, b = c.alloc_slot(), c.alloc_slot()
    c.prepare([a, b], [4, 4])
    st[a] = 1.0
    st[b] = 2.0
    c.commit([a, b], [4, 4])
    c.prepare([a, b], [1, 1])                # going on: state stays
    assert float(st[a].sum()) == 3.0 and float(st[b].sum()) == 6.0
    c.commit([a, b], [1, 1])
    c.free_slot(a)
    a2 = c.alloc_slot()
    assert a2 == a
    c.prepare([a2], [2])                     # a sequence that starts begins with zeros
    assert float(st[a2].abs().sum()) == 0.0 and float(st[b].sum()) == 6.0
    with pytest.raises(InvalidArgument, match="cannot be rewound"):
        c.commit([a2], [2]) or c.truncate(a2, 1)


def test_truncate():
    c = make()
    s = c.alloc_slot()
    c.prepare([s], [100])
    c.commit([s], [100])
    c.truncate(s, 60)
    assert c.length(s) == 60
    with pytest.raises(InvalidArgument):
        c.truncate(s, 61)


def test_random_walk_keeps_invariants():
    rng = random.Random(0)
    c = make(max_tokens=PAGE * 12, window=70)
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and c.slots.n_free:
            live[c.alloc_slot()] = 0
        elif op < 0.4 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            group = rng.sample(list(live), rng.randint(1, len(live)))
            n_new = [rng.choice([1, 1, 1, 17, 64, 130]) for _ in group]
            try:
                c.prepare(group, n_new)
            except ContextFull:
                c.check()
                continue
            c.commit(group, n_new)
            for s, n in zip(group, n_new):
                live[s] += n
        c.check()
        assert all(c.length(s) == n for s, n in live.items())
    for s in list(live):
        c.free_slot(s)
    c.check()
    assert all(g.pool.n_held == 0 for g in c.groups) and c.slots.n_held == 0


def test_sizes():
    c = Cache([(KVRequest(8, 128), None)] * 36, [None] * 36, 4096, torch.bfloat16, "meta")
    assert c.bytes() == 4096 * 2 * 36 * 8 * 128 * 2  # 147456 bytes per token at the 8B sizes
    assert c.n_pages == 64 and c.n_slots == 64
    assert Cache([(KVRequest(1, 16), None)], [None], 65, torch.float32, "cpu").max_tokens == 128
    with pytest.raises(InvalidArgument):
        Cache([(KVRequest(1, 16), None)], [None], 0, torch.float32, "cpu")


def test_rollback_undoes_a_prepare_whose_step_did_not_happen():
    c = make()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.prepare([a], [70])
    c.commit([a], [70])
    before = (c.groups[0].pool.n_free, {s: list(t) for s, t in c.groups[0].tables.items()})
    c.prepare([a, b], [PAGE * 2, 10])          # a grows by two pages, b takes its first
    assert c.groups[0].pool.n_free == before[0] - 3
    c.rollback([a, b])
    assert (c.groups[0].pool.n_free, {s: list(t) for s, t in c.groups[0].tables.items()}) == before
    c.check()
    c.prepare([a, b], [1, 1])                  # and the cache goes on as if nothing had been
    c.commit([a, b], [1, 1])
    assert c.length(a) == 71 and c.length(b) == 1
    c.check()
