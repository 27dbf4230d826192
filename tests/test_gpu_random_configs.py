"""Random tiny configurations and random traces against the plain implementation: head sizes in steps of 16,
any number of heads and groups, widths and vocabularies that are no power of two, windows on some layers,
biases, tied or untied output; batches of unequal prompts (some longer than 512 tokens), a cut in the middle
of a prompt, decoding with early leavers.  Seeds are fixed: the same cases every run."""
import numpy as np
import pytest
import torch

from gpu_util import TOL, check
from nncpu_b200 import Engine, Model
from plain_qwen3 import PlainQwen3
from tiny import make_folder

pytestmark = pytest.mark.gpu


def random_config(rs):
    hd = int(rs.choice([16, 32, 48, 64, 80, 96, 112, 128]))
    n_kv = int(rs.choice([1, 2, 3, 4]))
    group = int(rs.choice([1, 2, 3, 4, 5, 8]))
    layers = int(rs.choice([1, 2, 3]))
    window = int(rs.choice([0, 0, 24, 70, 150, 300]))
    types = [("sliding_attention" if window and rs.rand() < 0.6 else "full_attention") for _ in range(layers)]
    return dict(num_hidden_layers=layers, hidden_size=int(rs.choice([72, 100, 136, 200, 256])),
                num_attention_heads=n_kv * group, num_key_value_heads=n_kv, head_dim=hd,
                intermediate_size=int(rs.choice([88, 90, 160, 264])), vocab_size=int(rs.randint(200, 600)),
                rope_theta=float(rs.choice([1e4, 5e5, 1e6])), rms_norm_eps=float(rs.choice([1e-6, 1e-5, 3e-6])),
                tie_word_embeddings=bool(rs.rand() < 0.5), attention_bias=bool(rs.rand() < 0.3),
                max_position_embeddings=4096, use_sliding_window=bool(window), sliding_window=window or None,
                layer_types=types, eos_token_id=None)


def random_lengths(rs):
    n = int(rs.choice([1, 2, 3, 4]))
    lens = [int(rs.choice([1, 2, 17, 40, 65, 130, 260])) for _ in range(n)]
    if rs.rand() < 0.5:
        lens[0] = int(rs.choice([513, 600, 700]))          # long enough for the prompt kernels
    return lens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_random_configuration_and_trace(tmp_path, seed, dtype):
    rs = np.random.RandomState(1000 + seed)
    cfg = random_config(rs)
    folder = make_folder(tmp_path / "m", "A", seed=seed, store_dtype=torch.float32 if dtype == "float32" else torch.bfloat16,
                         **cfg)
    plain = PlainQwen3(folder)
    model = Model.load(folder, dtype=dtype)
    lens = random_lengths(rs)
    n_decode = [int(rs.randint(0, 12)) for _ in lens]
    reqs = [rs.randint(0, plain.cfg.vocab, size=n + d).tolist() for n, d in zip(lens, n_decode)]
    want = [plain.logits(r) for r in reqs]
    pages = sum((len(r) + 63) // 64 for r in reqs) + 2
    engine = Engine(model, max_tokens=64 * pages)
    for round_ in range(2):                                  # twice: the second time on reused slots and pages
        slots = [engine.alloc_slot() for _ in reqs]
        got = [[] for _ in reqs]
        # the prompts, the first one cut in two steps when it is long enough
        cut = lens[0] // 2 if lens[0] > 40 and round_ == 1 else 0
        if cut:
            out = engine.step([slots[0]], [reqs[0][:cut]], [list(range(cut))])
            got[0].append(out.clone())
            first = [reqs[0][cut:lens[0]]] + [r[:n] for r, n in zip(reqs[1:], lens[1:])]
        else:
            first = [r[:n] for r, n in zip(reqs, lens)]
        out = engine.step(slots, first, [list(range(len(t))) for t in first])
        at = 0
        for i, t in enumerate(first):
            got[i].append(out[at:at + len(t)].clone())
            at += len(t)
        step = 0
        while True:
            live = [i for i in range(len(reqs)) if step < n_decode[i]]
            for i in range(len(reqs)):
                if i not in live and slots[i] is not None:
                    engine.free_slot(slots[i])
                    slots[i] = None
            if not live:
                break
            out = engine.step([slots[i] for i in live], [[reqs[i][lens[i] + step]] for i in live])
            for row, i in enumerate(live):
                got[i].append(out[row:row + 1].clone())
            step += 1
        for i in range(len(reqs)):
            check(torch.cat(got[i]), want[i], TOL[dtype], f"seed {seed}, round {round_}, request {i} of {lens}, {cfg}")
        engine.cache.check()
    model.rt.check_status()
