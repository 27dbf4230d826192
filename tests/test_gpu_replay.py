"""bin/trace_run as a user runs it: a subprocess fed JSON steps on standard
input, logits read back from the files it writes, compared with the plain
implementation: whole requests, the last 32 tokens one by one, and batches of
unequal lengths one after another."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT
from gpu_util import TOL, check
from plain_qwen3 import PlainQwen3
from tiny import make_folder

pytestmark = pytest.mark.gpu


def replay(folder, dtype, steps, out, max_tokens):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(max_tokens)], input=text, capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    return p


def read(out, step, vocab):
    return np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, vocab)


@pytest.mark.parametrize("dtype,name", [("float32", "B"), ("bfloat16", "C")])
def test_replay(tmp_path, dtype, name):
    folder = make_folder(tmp_path / "m", name, seed=9,
                         store_dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    plain = PlainQwen3(folder)
    V = plain.cfg.vocab
    rs = np.random.RandomState(0)
    reqs = {k: rs.randint(0, V, size=n).tolist() for k, n in
            (("whole", 100), ("cut", 100), ("a", 20), ("b", 75), ("c", 8), ("d", 140), ("e", 33))}
    reqs["cut"] = list(reqs["whole"])
    want = {k: plain.logits(v) for k, v in reqs.items()}
    steps, expect = [], {}      # expect[step] = list of (request, positions)

    def add(entries, end=()):
        n = len(steps)
        steps.append({"step": n, "entries": [{"id": k, "tokens": reqs[k][a:b], "want": w} for k, a, b, w in entries],
                      "end": list(end)})
        if any(w for *_, w in entries):
            expect[n] = [(k, [a + i for i in w]) for k, a, b, w in entries if w]
    # each request alone and whole, every position wanted
    add([("whole", 0, 100, list(range(100)))], end=["whole"])
    # the same tokens with the last 32 one by one
    add([("cut", 0, 68, list(range(68)))])
    for t in range(68, 100):
        add([("cut", t, t + 1, [0])], end=["cut"] if t == 99 else [])
    # a batch of unequal lengths: prompts in one step, then one token each; shorter requests end earlier
    prompt = {"a": 12, "b": 70, "c": 3}
    add([(k, 0, prompt[k], [prompt[k] - 1] if k != "b" else [0, 69]) for k in "abc"])
    for i in range(8):
        live = [k for k in "abc" if prompt[k] + i < len(reqs[k])]
        add([(k, prompt[k] + i, prompt[k] + i + 1, [0] if (i + ord(k)) % 3 else []) for k in live],
            end=[k for k in live if prompt[k] + i + 1 == len(reqs[k])])
    # the next batch reuses what the first gave back
    add([("d", 0, 130, [129]), ("e", 0, 30, [29, 0])])
    for i in range(3):
        add([("d", 130 + i, 131 + i, [0]), ("e", 30 + i, 31 + i, [0])])
    add([("d", 133, 140, [6, 0])], end=["d", "e"])
    out = tmp_path / "out"
    # live tokens at any time, each request rounded up to 64: the first batch holds 64 + 128 + 64
    replay(folder, dtype, steps, out, max_tokens=64 * 4)
    assert sorted(int(p.stem) for p in out.glob("*.f32")) == sorted(expect)
    for n, items in expect.items():
        got = read(out, n, V)
        ref = np.concatenate([want[k][pos] for k, pos in items])
        check(got, ref, TOL[dtype], f"step {n}")
    # cutting the same tokens differently changes nothing beyond rounding
    whole = read(out, 0, V)
    cut = np.concatenate([read(out, 1, V)] + [read(out, n, V) for n in range(2, 34)])
    check(cut, whole, 1e-5 if dtype == "float32" else TOL[dtype], "whole against cut")


def test_replay_reports_a_full_cache(tmp_path):
    folder = make_folder(tmp_path / "m", "A", seed=1)
    step = {"step": 0, "entries": [{"id": "x", "tokens": [1] * 65, "want": []}], "end": []}
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "64"], input=json.dumps(step) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode != 0 and "ContextFull" in p.stderr
