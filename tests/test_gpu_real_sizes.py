"""The engine against the plain implementation at the layer sizes of Qwen3-8B, 14B and 32B (hidden size, heads,
head size, intermediate size and vocabulary as published; one layer of the 36, 40 and 64, as each test's id
says), in float32 and in bfloat16: sizes at which the tensor-core kernels run their real tile counts (K of
4 096 to 25 600, 32 to 64 heads, 151 936 output rows), which the tiny configurations cannot show.

The weights are drawn once per size on the device, written to a temporary model folder, and read from there by
both sides.  The plain side only computes the output rows that are compared."""
import numpy as np
import pytest
import torch

import plain_qwen3 as P
from gpu_util import DEV, TOL, check
from nncpu_b200 import Engine, Model
from nncpu_b200.config import config_from_dict
from nncpu_b200.engine.model import parameter_list
from nncpu_b200.weights import random_tensors_on_device, write_safetensors

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen3ForCausalLM"], num_key_value_heads=8, head_dim=128, vocab_size=151936,
            rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=False,
            max_position_embeddings=40960, num_hidden_layers=1)
SIZES = {   # name: (layers of the published model, its layer sizes)
    "8b": (36, dict(hidden_size=4096, num_attention_heads=32, intermediate_size=12288)),
    "14b": (40, dict(hidden_size=5120, num_attention_heads=40, intermediate_size=17408)),
    "32b": (64, dict(hidden_size=5120, num_attention_heads=64, intermediate_size=25600)),
}
IDS = {name: f"{name}-sizes-1-of-{layers}-layers" for name, (layers, _) in SIZES.items()}


@pytest.fixture(scope="module")
def made(tmp_path_factory):
    """size -> (folder, plain model with its layer matrices widened once)."""
    cache = {}

    def get(name):
        if name not in cache:
            cache.clear()                                    # one size's files and arrays at a time
            import json
            folder = tmp_path_factory.mktemp(f"qwen3_{name}")
            cfg = config_from_dict(dict(BASE, **SIZES[name][1]))
            (folder / "config.json").write_text(json.dumps(cfg.to_dict()))
            tensors = random_tensors_on_device(parameter_list(cfg.model_spec()), 7, torch.bfloat16, DEV)
            write_safetensors(folder / "model.safetensors", {k: v.cpu() for k, v in tensors.items()})
            del tensors
            torch.cuda.empty_cache()
            plain = P.PlainQwen3(folder)
            for k in list(plain.w):
                if "layers" in k and plain.w[k].ndim == 2:
                    plain.w[k] = plain.w[k].astype(np.float64)     # widened once, not at every product
            cache[name] = (folder, plain)
        return cache[name]
    return get


def plain_rows(plain, requests):
    """Logits of (tokens, rows) requests through one product with the output matrix."""
    hidden = [plain.hidden(toks)[list(rows)] for toks, rows in requests]
    return P.linear(np.concatenate(hidden), plain.w["lm_head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_of_20_and_70_on_the_same_pages(made, dtype):
    """At the 8B layer sizes: 20 prompts of unequal lengths decoded 4 steps (few-token products give way to the
    17-to-64-token ones), then, on the pages they gave back, 70 prompts (65-to-256-token products)."""
    folder, plain = made("8b")
    model = Model.load(folder, dtype=dtype)
    engine = Engine(model, max_tokens=64 * 80)
    rs = np.random.RandomState(2)
    for n_seqs, n_checked in ((20, 20), (70, 12)):
        lens = rs.randint(1, 41, size=n_seqs).tolist()
        reqs = [rs.randint(0, 151936, size=n + 4).tolist() for n in lens]
        slots = [engine.alloc_slot() for _ in reqs]
        got = [engine.step(slots, [r[:n] for r, n in zip(reqs, lens)]).clone()]
        for step in range(4):
            got.append(engine.step(slots, [[r[n + step]] for r, n in zip(reqs, lens)]).clone())
        got = torch.stack(got, dim=1)                                    # [sequence, step, vocab]
        picked = sorted(set(rs.choice(n_seqs, size=n_checked, replace=False).tolist())
                        | {int(np.argmin(lens)), int(np.argmax(lens))})
        want = plain_rows(plain, [(reqs[i], range(lens[i] - 1, lens[i] + 4)) for i in picked])
        check(got[picked].reshape(-1, 151936), want, TOL[dtype], f"{IDS['8b']}, {dtype}: batch of {n_seqs}")
        for s in slots:
            engine.free_slot(s)
        engine.cache.check()
        assert all(g.pool.n_held == 0 for g in engine.cache.groups)
    model.rt.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SIZES), ids=[IDS[n] for n in SIZES])
def test_long_prompt_whole_and_with_its_last_32_tokens_one_by_one(made, name, dtype):
    folder, plain = made(name)
    model = Model.load(folder, dtype=dtype)
    engine = Engine(model, max_tokens=64 * 24)
    toks = np.random.RandomState(1).randint(0, 151936, size=600).tolist()
    places = [0, 63, 64, 127, 128, 300, 511, 512, 567] + list(range(568, 600))
    want = plain_rows(plain, [(toks, places)])
    s = engine.alloc_slot()
    whole = engine.step([s], [toks], [places]).clone()      # a step's result is valid until the next step
    check(whole, want, TOL[dtype], f"{IDS[name]}, {dtype}: 600 tokens whole")
    engine.free_slot(s)
    s = engine.alloc_slot()
    head = engine.step([s], [toks[:568]], [places[:9]]).clone()
    tail = [engine.step([s], [[t]]).clone() for t in toks[568:]]
    cut = torch.cat([head] + tail)
    check(cut, want, TOL[dtype], f"{IDS[name]}, {dtype}: the last 32 tokens one by one")
    check(cut, whole, 2e-5 if dtype == "float32" else TOL[dtype], "cut against whole")
    model.rt.check_status()
