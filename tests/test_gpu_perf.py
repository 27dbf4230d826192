"""The phase profiler on the device: its phases add up to the step they cut up, its byte model is the
model's own, and switching it on changes no result."""
import numpy as np
import pytest
import torch

import nncpu_b200
from gpu_util import check
from nncpu_b200 import Engine, Model, perf_enable, perf_report, perf_reset, perf_span_ms, perf_totals
from tiny import make_folder

pytestmark = pytest.mark.gpu

PRODUCTS = ("attn_qkv", "attn_out", "ffn_gate_up", "ffn_down", "lm_head")


@pytest.fixture(autouse=True)
def profiler_off_afterwards():
    yield
    perf_enable(False)
    perf_reset()


@pytest.mark.parametrize("dtype,hidden", [("bfloat16", 2048), ("float32", 1024)])
def test_phases_add_up_and_count_the_models_bytes(dtype, hidden):
    # wide enough that the device, not the host's launches, sets the prompt step's time in either element type
    from tiny import tiny_config
    cfg = tiny_config("G", hidden_size=hidden, intermediate_size=4 * hidden, num_attention_heads=hidden // 128,
                      num_key_value_heads=4, vocab_size=32000, num_hidden_layers=4, layer_types=None,
                      use_sliding_window=False)
    model = Model.random(cfg, seed=3, dtype=dtype)
    engine = Engine(model, max_tokens=64 * 300)
    rs = np.random.RandomState(0)
    lens = (2000, 2100, 1800, 2011) if dtype == "float32" else (4000, 4200, 4600, 4011, 1500)
    prompts = [rs.randint(0, 32000, size=n).tolist() for n in lens]
    slots = [engine.alloc_slot() for _ in prompts]
    plain_prefill = engine.step(slots, prompts).clone()
    nxt = [[int(t)] for t in plain_prefill.argmax(-1)]
    plain_decode = engine.step(slots, nxt).clone()           # through the graph
    for s in slots:
        engine.free_slot(s)
    slots = [engine.alloc_slot() for _ in prompts]
    perf_enable(True)
    perf_reset()
    a, b, c, d = (torch.cuda.Event(enable_timing=True) for _ in range(4))
    torch.cuda.synchronize()
    a.record()
    got_prefill = engine.step(slots, prompts).clone()
    b.record()
    prefill, prefill_span = perf_totals(), perf_span_ms()
    perf_reset()
    n_decode = 5
    c.record()
    for _ in range(n_decode):
        got_decode = engine.step(slots, nxt)                 # kernel by kernel while the profiler is on
        for s in slots:
            engine.cache.truncate(s, engine.cache.length(s) - 1)
    d.record()
    decode = perf_totals()
    torch.cuda.synchronize()
    # switching the profiler on changes no result (the decode step leaves its graph for single kernels)
    assert torch.equal(got_prefill, plain_prefill)
    check(got_decode, plain_decode, 1e-5 if dtype == "float32" else 2e-2, "decode step kernel by kernel")
    # The slots cut the step up.  From the first kernel to the last they leave out only the seams between scopes
    # (within a tenth); the event-timed step around the call also holds the host's work before the first kernel.
    prefill_ms, step_ms = sum(t["ms"] for t in prefill.values()), a.elapsed_time(b)
    assert 0.9 * prefill_span <= prefill_ms <= 1.001 * prefill_span <= 1.002 * step_ms, (prefill_ms, prefill_span, step_ms)
    decode_ms, loop_ms = sum(t["ms"] for t in decode.values()), c.elapsed_time(d)
    assert decode_ms <= 1.001 * loop_ms, (decode_ms, loop_ms)
    # every product phase streamed its weights once per step
    assert sum(decode[k]["bytes"] for k in PRODUCTS) == n_decode * model.weight_bytes_per_step()
    assert sum(prefill[k]["bytes"] for k in PRODUCTS) == model.weight_bytes_per_step()
    assert decode["attn_qkv"]["calls"] == n_decode * 4 and decode["lm_head"]["calls"] == n_decode
    # in bfloat16 the few-token products carry the norms between them: only the first and the final norm are launches
    assert decode["norm"]["calls"] == n_decode * (2 if dtype == "bfloat16" else 9) and decode["embed"]["calls"] == n_decode
    # attention counts, per token, the keys and values of its span
    spec = model.spec.layers[0].mixer
    row = 2 * spec.n_kv_heads * spec.head_dim * (2 if dtype == "bfloat16" else 4)
    spans = sum(n * (n + 1) // 2 for n in lens)
    assert prefill["attn_core"]["bytes"] == 4 * spans * row
    assert decode["attn_core"]["bytes"] == n_decode * 4 * sum(n + 1 for n in lens) * row
    assert decode["attn_core"]["flops"] == n_decode * 4 * 4.0 * sum(n + 1 for n in lens) * \
        spec.n_heads * spec.head_dim
    text = perf_report("decode", n_tokens=4 * n_decode, peaks={"hbm_gbs": 6552.0, "bf16_tflops": 1628.5})
    assert "ffn_gate_up" in text and "of peak" in text and "ms/token over 20 tokens" in text
    model.rt.check_status()


def test_phase_table_from_the_command_line(tmp_path):
    import subprocess
    import sys
    from conftest import ROOT
    folder = make_folder(tmp_path / "m", "A", seed=1)
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "nncpu-b200"), "--gen", str(folder), "5 6 7 8", "12",
                        "--fp32", "--perf"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "nncpu perf - gen" in p.stdout and "attn_core" in p.stdout and "lm_head" in p.stdout
    assert "ms/token over 16 tokens" in p.stdout
    assert nncpu_b200.perf_report("x").endswith("no samples\n")
