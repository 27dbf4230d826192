"""The whole model through the engine's step function against the plain
implementation, in float32 and in bfloat16: each request alone and whole; the
last 32 tokens one by one; batches of unequal lengths whose shorter requests
end earlier, one batch after another on reused slots; long decoding; the first
tokens of a sequence; and weights made so that a far key, a window's edge or a
stale cache row would show."""
import numpy as np
import pytest
import torch

from gpu_util import TOL, check
from nncpu_b200 import Engine, Model
from nncpu_b200.errors import ContextFull, InvalidArgument
from nncpu_b200.weights import SafetensorsFile, write_safetensors
from plain_qwen3 import PlainQwen3
from tiny import make_folder

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
# bfloat16 models are compared with a reference that reads the same (rounded) weights
STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    out = {}
    for name in "ABCDEFG":
        for dtype in DTYPES:
            out[name, dtype] = make_folder(root / f"{name}_{dtype}", name, seed=ord(name), store_dtype=STORE[dtype])
    return out


@pytest.fixture(scope="module")
def plains(folders):
    return {key: PlainQwen3(folder) for key, folder in folders.items()}


def tokens_for(plain, n, seed):
    return np.random.RandomState(seed).randint(0, plain.cfg.vocab, size=n).tolist()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", "ABCDEFG")
def test_whole_then_last_32_one_by_one(folders, plains, name, dtype):
    plain = plains[name, dtype]
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 16)
    toks = tokens_for(plain, 150, 1)
    want = plain.logits(toks)
    s = engine.alloc_slot()
    whole = engine.step([s], [toks], [list(range(150))]).clone()      # a step's result is valid until the next step
    check(whole, want, TOL[dtype], "whole request")
    s2 = engine.alloc_slot()
    head = engine.step([s2], [toks[:118]], [list(range(118))]).clone()
    tail = [engine.step([s2], [[t]]).clone() for t in toks[118:]]
    cut = torch.cat([head] + tail)
    check(cut, want, TOL[dtype], "last 32 tokens one by one")
    # how the tokens are cut changes nothing beyond rounding
    check(cut, whole, 1e-5 if dtype == "float32" else TOL[dtype], "cut against whole")
    model.rt.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", "ABCDEFG")
def test_unequal_batches_one_after_another(folders, plains, name, dtype):
    plain = plains[name, dtype]
    model = Model.load(folders[name, dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 8)      # small: the second batch must reuse pages
    for round_, lens in enumerate(([1, 7, 17, 30, 70], [66, 3, 129], [5, 9, 13])):
        n_decode = [3, 12, 6, 9, 1][:len(lens)]      # shorter requests end earlier
        reqs = [tokens_for(plain, n + d, 100 * round_ + i) for i, (n, d) in enumerate(zip(lens, n_decode))]
        want = [plain.logits(r) for r in reqs]
        slots = [engine.alloc_slot() for _ in reqs]
        got = [[] for _ in reqs]
        out = engine.step(slots, [r[:n] for r, n in zip(reqs, lens)], [list(range(n)) for n in lens])
        at = 0
        for i, n in enumerate(lens):
            got[i].append(out[at:at + n].clone())
            at += n
        live = list(range(len(reqs)))
        step = 0
        while live:
            live = [i for i in live if step < n_decode[i]]
            for i in range(len(reqs)):
                if i not in live and slots[i] is not None and step >= n_decode[i]:
                    engine.free_slot(slots[i])
                    slots[i] = None
            if not live:
                break
            out = engine.step([slots[i] for i in live], [[reqs[i][lens[i] + step]] for i in live])
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1].clone())
            step += 1
        for i in range(len(reqs)):
            check(torch.cat(got[i]), want[i], TOL[dtype], f"batch {round_}, request {i} of lengths {lens}")
        engine.cache.check()
        assert engine.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in engine.cache.groups)
    model.rt.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompts_whole_cut_and_batched(folders, plains, dtype):
    """Prompts of more than 512 tokens: in bfloat16 the q/k/v projection runs with its fused epilogue and
    attention on 128-row tiles.  A request whole, the same request cut into a long and a short step and
    then decoded, and two long requests of unequal lengths in one batch all agree with the plain model."""
    plain = plains["G", dtype]
    model = Model.load(folders["G", dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 40)
    a, b = tokens_for(plain, 700, 11), tokens_for(plain, 530, 12)
    want_a, want_b = plain.logits(a), plain.logits(b)
    places = sorted(set(range(0, 700, 37)) | {127, 128, 255, 256, 511, 512, 639, 640, 699})
    s = engine.alloc_slot()
    whole = engine.step([s], [a], [places]).clone()      # a step's result is valid until the next step
    check(whole, want_a[places], TOL[dtype], "whole request")
    engine.free_slot(s)
    s = engine.alloc_slot()
    head = engine.step([s], [a[:560]], [[p for p in places if p < 560]]).clone()
    mid = engine.step([s], [a[560:690]], [[p - 560 for p in places if 560 <= p < 690]]).clone()
    tail = torch.cat([engine.step([s], [[t]]).clone() for t in a[690:]])
    cut = torch.cat([head, mid])
    n_cut = cut.shape[0]
    check(cut, want_a[[p for p in places if p < 690]], TOL[dtype], "cut into 560 + 130")
    check(tail, want_a[690:], TOL[dtype], "then one by one")
    check(cut, whole[:n_cut], 1e-5 if dtype == "float32" else TOL[dtype], "cut against whole")
    engine.free_slot(s)
    s1, s2 = engine.alloc_slot(), engine.alloc_slot()
    both = engine.step([s1, s2], [a, b], [[0, 300, 699], [0, 529]])
    check(both[:3], want_a[[0, 300, 699]], TOL[dtype], "batched, first request")
    check(both[3:], want_b[[0, 529]], TOL[dtype], "batched, second request")
    model.rt.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_reused_slots_with_other_pages_and_the_same_lengths(folders, plains, dtype):
    """Two pairs of requests of the same lengths, one after the other in the same slots.  The second pair's
    prompts run in the other order, so the slots hold other pages while every length is what it was: a
    decode step that remembered the first pair's page tables would read the first pair's keys."""
    plain = plains["B", dtype]
    model = Model.load(folders["B", dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 8)
    for round_ in range(2):
        a, b = tokens_for(plain, 70 + 6, 21 + 10 * round_), tokens_for(plain, 130 + 6, 22 + 10 * round_)
        want_a, want_b = plain.logits(a), plain.logits(b)
        slots = sorted([engine.alloc_slot(), engine.alloc_slot()])
        if round_ == 0:
            engine.step(slots, [a[:70], b[:130]])
        else:
            engine.step([slots[1]], [b[:130]])
            engine.step([slots[0]], [a[:70]])
        got_a, got_b = [], []
        for i in range(6):
            out = engine.step(slots, [[a[70 + i]], [b[130 + i]]])
            got_a.append(out[0:1].clone())
            got_b.append(out[1:2].clone())
        check(torch.cat(got_a), want_a[70:], TOL[dtype], f"round {round_}, first request")
        check(torch.cat(got_b), want_b[130:], TOL[dtype], f"round {round_}, second request")
        for s_ in slots:
            engine.free_slot(s_)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(folders, plains, dtype):
    plain = plains["B", dtype]
    model = Model.load(folders["B", dtype], dtype=dtype)
    engine = Engine(model, max_tokens=64 * 8)
    toks = tokens_for(plain, 200, 5)
    want = plain.logits(toks)
    s = engine.alloc_slot()
    got = [engine.step([s], [[t]]).clone() for t in toks]      # from the very first token, one by one
    got = torch.cat(got)
    check(got[:4], want[:4], TOL[dtype], "the first tokens of a sequence")
    check(got, want, TOL[dtype], "200 tokens decoded one by one")
    assert engine.cache.length(s) == 200


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", "ACDE")
def test_sharp_attention_shows_far_keys_window_edges_and_stale_rows(folders, name, dtype, tmp_path):
    """Random weights give nearly flat attention, under which a wrong far key
    or a stale cache row barely moves the logits.  Scaling the per-head q norm
    weights makes the softmax peaked, so single keys decide the output."""
    f = SafetensorsFile(folders[name, dtype] / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    for n in tensors:
        if n.endswith("q_norm.weight"):
            tensors[n] = (tensors[n].float() * 6.0).to(tensors[n].dtype)
    folder = tmp_path / "sharp"
    folder.mkdir()
    (folder / "config.json").write_text((folders[name, dtype] / "config.json").read_text())
    write_safetensors(folder / "model.safetensors", tensors)
    # Peaked attention also amplifies the rounding of q and k to bfloat16 itself; so that the comparison
    # measures the kernels and not the format, the bfloat16 oracle rounds its activations at the same places.
    plain = PlainQwen3(folder, round_activations_to_bf16=(dtype == "bfloat16"))
    model = Model.load(folder, dtype=dtype)
    engine = Engine(model, max_tokens=64 * 12)
    tol = TOL[dtype]
    # a long request fills the pages; it ends; a short one reuses slot and pages and must not see its rows
    long_ = tokens_for(plain, 400, 7)
    s = engine.alloc_slot()
    out = engine.step([s], [long_], [[399, 398, 200]])
    want = plain.logits(long_)
    check(out, want[[399, 398, 200]], tol, "far keys among hundreds")
    engine.free_slot(s)
    short = tokens_for(plain, 70, 8)
    s = engine.alloc_slot()
    got = torch.cat([engine.step([s], [short[:40]], [list(range(40))]).clone()] +
                    [engine.step([s], [[t]]).clone() for t in short[40:]])
    check(got, plain.logits(short), tol, "a reused slot")
    # two slots with the same tokens agree exactly, wherever their pages lie
    s2, s3 = engine.alloc_slot(), engine.alloc_slot()
    both = engine.step([s2, s3], [short, short], [[69], [69]])
    assert torch.equal(both[0], both[1])


def test_step_refuses_bad_arguments_before_changing_anything(folders):
    model = Model.load(folders["A", "float32"], dtype="float32")
    engine = Engine(model, max_tokens=128, max_seq_len=100)
    s = engine.alloc_slot()
    engine.step([s], [[1, 2, 3]])
    for bad in (lambda: engine.step([s], [[256]]), lambda: engine.step([s], [[-1]]),
                lambda: engine.step([s], [[]]), lambda: engine.step([s], [[1]], [[1]]),
                lambda: engine.step([s, s], [[1], [2]]), lambda: engine.step([5], [[1]]),
                lambda: engine.step([], [])):
        with pytest.raises(InvalidArgument):
            bad()
    with pytest.raises(ContextFull):
        engine.step([s], [[1] * 98])
    assert engine.cache.length(s) == 3
    engine.cache.check()
    assert engine.step([s], [[4]], [[]]) is None and engine.cache.length(s) == 4


def test_stored_32_bit_tensors_stay_32_bit_in_a_bfloat16_run(tmp_path):
    folder = make_folder(tmp_path / "m", "B", seed=3, store_dtype=torch.bfloat16, vector_dtype=torch.float32)
    model = Model.load(folder, dtype="bfloat16")
    assert model.blocks[0].norm1.gamma.dtype == torch.float32
    assert model.blocks[0].mixer.q_gamma.dtype == torch.float32 and model.blocks[0].mixer.b_qkv.dtype == torch.float32
    assert model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    plain = PlainQwen3(folder)
    toks = tokens_for(plain, 40, 2)
    engine = Engine(model, max_tokens=64)
    s = engine.alloc_slot()
    check(engine.step([s], [toks], [list(range(40))]), plain.logits(toks), TOL["bfloat16"], "mixed element types")
    # all-float32 file in a bfloat16 run: the matrices stay float32 and run on the 32-bit kernels
    folder = make_folder(tmp_path / "f", "A", seed=3, store_dtype=torch.float32)
    model = Model.load(folder, dtype="bfloat16")
    assert model.blocks[0].mixer.w_qkv.dtype == torch.float32
    plain = PlainQwen3(folder)
    toks = tokens_for(plain, 40, 2)
    engine = Engine(model, max_tokens=64)
    s = engine.alloc_slot()
    check(engine.step([s], [toks[:20]], [list(range(20))]), plain.logits(toks[:20]), TOL["bfloat16"], "float32 file")


def test_float32_cache_in_a_bfloat16_run(folders, plains):
    model = Model.load(folders["A", "bfloat16"], dtype="bfloat16")
    engine = Engine(model, max_tokens=128, kv_dtype=torch.float32)
    assert engine.cache.groups[0].k.dtype == torch.float32
    toks = tokens_for(plains["A", "bfloat16"], 50, 3)
    s = engine.alloc_slot()
    check(engine.step([s], [toks], [list(range(50))]), plains["A", "bfloat16"].logits(toks), TOL["bfloat16"], "kv f32")


def test_position_range_of_the_config_sets_only_the_default_context(tmp_path):
    """max_position_embeddings is the default context of a session (crates/nncpu/src/session/engine.rs:113-117);
    the engine itself runs a sequence as far as its cache reaches."""
    from nncpu_b200 import Session, SessionParams
    folder = make_folder(tmp_path / "m", "A", seed=5, max_position_embeddings=64)
    plain = PlainQwen3(folder)
    model = Model.load(folder, dtype="float32")
    engine = Engine(model, max_tokens=256)
    toks = tokens_for(plain, 150, 9)
    s = engine.alloc_slot()
    got = torch.cat([engine.step([s], [toks[:100]], [list(range(100))]).clone()] +
                    [engine.step([s], [[t]]).clone() for t in toks[100:]])
    check(got, plain.logits(toks), TOL["float32"], "beyond the configured position range")
    assert Session(model).n_ctx == 64 and Session(model, SessionParams(n_ctx=300)).n_ctx == 300
