#!/usr/bin/env python3
"""Benchmark of the library's flagship step: decoding with the Qwen3-8B layer
sizes, random weights, bfloat16, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a batch of 8 sequences whose prompts are 2,048
tokens long (context length 4,096).  ``value`` is decoded tokens per second,
timed on the device with CUDA events over exactly K steps after W warm-up
steps; by default K extends the prompts to the full context (2,039 steps after
8 warm-up steps).  ``e2e`` is the same workload through ``Session.generate``
with host token ids in and out.  The line also carries a prefill measurement (one
2,048-token prompt), the decode step's memory roofline, decode at batch 1 and
64, and the SM clocks sampled during the timed region.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
                rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=False,
                max_position_embeddings=40960)
# The larger layer sizes of the benchmark description, for `--model 14b|32b` (not the default run).
SIZES = {
    "8b": {},
    "14b": dict(num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600),
}
CONTEXT = 4096
PROMPT = 2048
BATCH = 8


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]),
                    # the burst figure: the prefill step is 25 ms of work timed on its own, not a seconds-long loop
                    "bf16_tflops": float(d.get("bf16_tflops") or d["bf16_tflops_sustained"]),
                    "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def sustained_tflops() -> float:
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["bf16_tflops_sustained"])
    except Exception:
        return 1400.0       # an earlier measurement on this pool: about 1.4 PFLOP/s at 1.3 GHz under the power cap


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def flops_prefill(cfg, T: int) -> float:
    """Multiply-adds times two of one T-token prompt: the layer matrices, causal
    attention (scores and weighted sum over half the square), one output row."""
    q = cfg.num_attention_heads * cfg.head_dim
    kv = cfg.num_key_value_heads * cfg.head_dim
    h, i = cfg.hidden_size, cfg.intermediate_size
    per_tok = 2.0 * (h * (q + 2 * kv) + q * h + 3 * h * i)
    attn = 4.0 * q * (T * (T + 1) / 2.0)
    return cfg.num_hidden_layers * (per_tok * T + attn) + 2.0 * h * cfg.vocab_size


def kv_bytes_per_token(cfg, esize: int = 2) -> int:
    return 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * esize


def timed_decode(engine, slots, first_tokens, steps: int, warmup: int):
    """W warm-up decode steps, then exactly K timed ones (greedy, token ids stay
    on the device).  Returns (milliseconds for K steps, mean kv length)."""
    import torch
    toks = engine.decode_run(slots, first_tokens, warmup) if warmup > 0 else None
    nxt = first_tokens if toks is None else toks[-1]
    torch.cuda.synchronize()
    lens0 = [engine.cache.length(s) for s in slots]
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    out = engine.decode_run(slots, nxt, steps)
    b.record()
    torch.cuda.synchronize()
    engine.model.rt.check_status()
    mean_len = sum(lens0) / len(lens0) + (steps + 1) / 2.0
    return a.elapsed_time(b), mean_len, out


def run_decode_point(model, cfg, batch: int, steps: int, warmup: int, seed: int = 0, with_phases: bool = False):
    import torch
    from nncpu_b200 import Engine
    per_seq = (CONTEXT + 63) // 64 * 64
    engine = Engine(model, max_tokens=per_seq * batch, max_seq_len=CONTEXT)
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, cfg.vocab_size, (batch, PROMPT), generator=g).tolist()
    slots = [engine.alloc_slot() for _ in range(batch)]
    # prefill in chunks of sequences to bound activation memory
    firsts = []
    from nncpu_b200.kernels import ops
    for i in range(0, batch, 4):
        logits = engine.step(slots[i:i + 4], prompts[i:i + 4])
        ids = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        ops.argmax(logits, ids)
        firsts += ids.tolist()
    steps = min(steps, CONTEXT - PROMPT - warmup - 1)
    ms, mean_len, _ = timed_decode(engine, slots, firsts, steps, warmup)
    tok_s = batch * steps / (ms / 1e3)
    bytes_step = model.weight_bytes_per_step() + batch * mean_len * kv_bytes_per_token(cfg)
    phases = None
    if with_phases:
        # the same engine, a few steps kernel by kernel under the phase profiler: where a step's time goes
        from nncpu_b200 import perf_enable, perf_reset, perf_totals
        for s in slots:      # the middle of the timed range, and in any case room for the steps below
            engine.cache.truncate(s, min(engine.cache.length(s), (PROMPT + CONTEXT) // 2, CONTEXT - 16))
        room = 9
        if room > 1:
            toks = [[1]] * batch
            engine.step(slots, toks)
            perf_enable(True)
            perf_reset()
            for _ in range(room - 1):
                engine.step(slots, toks)
            phases = {k: round(v["ms"] / (room - 1), 4) for k, v in perf_totals().items()}
            perf_enable(False)
            perf_reset()
    for s in slots:
        engine.free_slot(s)
    del engine
    torch.cuda.empty_cache()
    return tok_s, ms / steps, bytes_step, (mean_len - (steps + 1) / 2.0 + 1, mean_len + (steps + 1) / 2.0 - 1), phases


def run_prefill(model, cfg, reps: int = 3):
    import torch
    from nncpu_b200 import Engine
    engine = Engine(model, max_tokens=PROMPT + 64, max_seq_len=CONTEXT)
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, cfg.vocab_size, (PROMPT,), generator=g).tolist()
    best = None
    for r in range(reps + 1):
        slot = engine.alloc_slot()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([slot], [prompt])
        b.record()
        torch.cuda.synchronize()
        engine.free_slot(slot)
        if r > 0:
            ms = a.elapsed_time(b)
            best = ms if best is None else min(best, ms)
    model.rt.check_status()
    del engine
    torch.cuda.empty_cache()
    return best


def run_e2e(model, cfg, steps: int, warmup: int):
    """The same decode workload through the public entry point: host token ids
    in, host token ids out, every step.  A first call of ``warmup`` steps on the
    same session is not timed (it builds the CUDA graph of this batch size)."""
    import torch
    from nncpu_b200 import GenerateParams, SamplerParams, Session, SessionParams
    session = Session(model, SessionParams(n_ctx=CONTEXT, seed=1, max_batch=BATCH))
    g = torch.Generator().manual_seed(3)
    prompts = torch.randint(0, cfg.vocab_size, (BATCH, PROMPT), generator=g).tolist()
    steps = min(steps, CONTEXT - PROMPT - 1)
    session.generate(prompts, GenerateParams(max_tokens=max(warmup, 1), sampler=SamplerParams.greedy()), stop_token_ids=())
    res = session.generate(prompts, GenerateParams(max_tokens=steps, sampler=SamplerParams.greedy()),
                           stop_token_ids=())
    n = sum(r.n_generated for r in res)
    decode_s = res[0].decode
    return {"value": n / decode_s if decode_s > 0 else None, "unit": "tokens/s",
            "h2d_bytes_per_step": session.engine.h2d_bytes_last_step, "d2h_bytes_per_step": 4 * BATCH,
            "prefill_s": res[0].prefill, "generated": n}


# The two larger workloads of the benchmark description, run through the public entry point, and a sweep of
# longer contexts than the contract's line covers.
WORKLOADS = {
    "14b-unequal": dict(model="14b", batch=16, prompt=(128, 2048), decode=256),
    "32b": dict(model="32b", batch=8, prompt=(2048, 2048), decode=512),
    "long-context": dict(model="8b"),
}


def run_long_context() -> dict:
    """Qwen3-8B sizes beyond the contract's 4 096 tokens: one prompt of 8 192 tokens, and decoding at batch 1 and 8
    with 16 384 and 32 768 keys per sequence (128 device-timed steps after 8 warm-up steps, greedy)."""
    import torch
    from nncpu_b200 import Engine, Model
    from nncpu_b200.config import config_from_dict
    from nncpu_b200.kernels import ops
    cfg = config_from_dict(dict(QWEN3_8B))
    model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    pk = peaks()
    out = {"workload": "long-context", "model": "Qwen3-8B sizes", "layers": cfg.num_hidden_layers, "dtype": "bf16",
           "peaks": pk["source"], "data": "synthetic: random weights, uniform random token ids"}
    g = torch.Generator().manual_seed(9)
    engine = Engine(model, max_tokens=8192 + 64, max_seq_len=8192 + 64, max_step_tokens=8192)
    prompt = torch.randint(0, cfg.vocab_size, (8192,), generator=g).tolist()
    best = None
    for r in range(3):
        slot = engine.alloc_slot()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([slot], [prompt])
        b.record()
        torch.cuda.synchronize()
        engine.free_slot(slot)
        if r > 0:
            best = a.elapsed_time(b) if best is None else min(best, a.elapsed_time(b))
    out["prefill_8192"] = {"ms": best, "value": 8192 / (best / 1e3),
                           "frac": flops_prefill(cfg, 8192) / (best / 1e3) / (pk["bf16_tflops"] * 1e12)}
    del engine
    torch.cuda.empty_cache()
    for ctx in (16384, 32768):
        for batch in (1, 8):
            engine = Engine(model, max_tokens=(ctx + 256) * batch, max_seq_len=ctx + 256, max_step_tokens=8192)
            slots = [engine.alloc_slot() for _ in range(batch)]
            firsts = []
            for s in slots:          # prompts go in one by one, 8 192 tokens a step
                toks = torch.randint(0, cfg.vocab_size, (ctx,), generator=g).tolist()
                for at in range(0, ctx, 8192):
                    logits = engine.step([s], [toks[at:at + 8192]])
                ids = torch.empty(1, dtype=torch.int32, device=logits.device)
                ops.argmax(logits, ids)
                firsts += ids.tolist()
            ms, mean_len, _ = timed_decode(engine, slots, firsts, 128, 8)
            step_bytes = model.weight_bytes_per_step() + batch * mean_len * kv_bytes_per_token(cfg)
            out[f"decode_b{batch}_ctx{ctx}"] = {"value": batch * 128 / (ms / 1e3), "ms_per_step": ms / 128,
                                                "hbm_frac": step_bytes / (ms / 128 / 1e3) / 1e9 / pk["hbm_gbs"]}
            for s in slots:
                engine.free_slot(s)
            del engine
            torch.cuda.empty_cache()
    return out


def run_workload(name: str) -> dict:
    """Batch of prompts (lengths uniform in the workload's range) through
    ``Session.generate``: one prefill step, then the workload's decode steps,
    greedy, host token ids in and out.  The first call (a few tokens) builds the
    CUDA graphs and is not timed."""
    import torch
    from nncpu_b200 import GenerateParams, Model, SamplerParams, Session, SessionParams
    from nncpu_b200.config import config_from_dict
    w = WORKLOADS[name]
    cfg = config_from_dict(dict(QWEN3_8B, **SIZES[w["model"]]))
    model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    g = torch.Generator().manual_seed(5)
    lo, hi = w["prompt"]
    lengths = torch.randint(lo, hi + 1, (w["batch"],), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lengths]
    session = Session(model, SessionParams(n_ctx=hi + w["decode"] + 1, seed=1, max_batch=w["batch"]))
    session.generate(prompts, GenerateParams(max_tokens=4, sampler=SamplerParams.greedy()), stop_token_ids=())
    res = session.generate(prompts, GenerateParams(max_tokens=w["decode"], sampler=SamplerParams.greedy()),
                           stop_token_ids=())
    n = sum(r.n_generated for r in res)
    mean_len = sum(lengths) / len(lengths) + w["decode"] / 2.0
    step_bytes = model.weight_bytes_per_step() + w["batch"] * mean_len * kv_bytes_per_token(cfg)
    step_s = res[0].decode / w["decode"]
    pk = peaks()
    return {"workload": name, "model": f"Qwen3-{w['model'].upper()} sizes", "layers": cfg.num_hidden_layers,
            "batch": w["batch"], "prompt_tokens": sum(lengths), "prompt_lengths": f"{min(lengths)}..{max(lengths)}",
            "decode_steps": w["decode"], "generated": n, "prefill_s": res[0].prefill,
            "prefill_tokens_per_s": sum(lengths) / res[0].prefill, "decode_s": res[0].decode,
            "decode_tokens_per_s": n / res[0].decode, "ms_per_step": step_s * 1e3,
            "hbm_frac": step_bytes / step_s / 1e9 / pk["hbm_gbs"], "peaks": pk["source"], "dtype": "bf16",
            "data": "synthetic: random weights, uniform random token ids"}


def fp32_check(cfg, name: str) -> dict:
    """The same random weights (rounded to bfloat16) run in bfloat16 and in true float32: how far the
    logits of a 96-token prompt, and of 8 tokens decoded after it, are apart."""
    import torch
    from nncpu_b200 import Engine, Model
    from nncpu_b200.engine.model import parameter_list
    from nncpu_b200.parts import Runtime
    from nncpu_b200.weights import random_tensors_on_device
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, cfg.vocab_size, (104,), generator=g).tolist()
    out = {}
    for dtype in ("bfloat16", "float32"):
        rt = Runtime("cuda:0", torch.bfloat16 if dtype == "bfloat16" else torch.float32)
        tensors = random_tensors_on_device(parameter_list(cfg.model_spec()), 0, torch.bfloat16, rt.device)
        if dtype == "float32":
            tensors = {k: v.float() for k, v in tensors.items()}
        model = Model(cfg, tensors, rt)
        del tensors
        engine = Engine(model, max_tokens=128)
        slot = engine.alloc_slot()
        rows = [engine.step([slot], [toks[:96]], [[0, 47, 95]]).clone()]
        rows += [engine.step([slot], [[t]]).clone() for t in toks[96:]]
        out[dtype] = torch.cat(rows).cpu()
        model.rt.check_status()
        del engine, model
        torch.cuda.empty_cache()
    diff = (out["bfloat16"] - out["float32"]).abs().max().item()
    scale = out["float32"].abs().max().item()
    agree = (out["bfloat16"].argmax(-1) == out["float32"].argmax(-1)).float().mean().item()
    return {"check": "bfloat16 against float32 logits", "model": f"Qwen3-{name.upper()} sizes",
            "layers": cfg.num_hidden_layers, "rows": out["float32"].shape[0], "max_abs_diff": diff,
            "max_abs_logit": scale, "relative": diff / scale, "same_top_token": agree}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=CONTEXT - PROMPT)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (named in config)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--model", default="8b", choices=sorted(SIZES), help="layer sizes (default: the benchmark's 8b)")
    ap.add_argument("--workload", choices=sorted(WORKLOADS),
                    help="instead of the contract's line: one of the description's larger workloads, end to end")
    ap.add_argument("--fp32-check", action="store_true",
                    help="instead of timing: logits of a short prompt in bfloat16 against the true 32-bit path")
    ap.add_argument("--no-launch-overlap", action="store_true",
                    help="for comparison: every kernel of a decode step waits for the end of the one before it")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "ZacWalk/nncpu is a Rust crate with no Python package and no Rust toolchain is installed: "
                          "pip cannot install it offline and it has no GPU path"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library is single-GPU by design, --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from nncpu_b200.config import config_from_dict
    from nncpu_b200 import Model
    from nncpu_b200.kernels import ops

    if args.no_launch_overlap:
        ops.launch_overlap(False)
    d = dict(QWEN3_8B, **SIZES[args.model])
    full_layers = d["num_hidden_layers"]
    if args.layers:
        d["num_hidden_layers"] = args.layers
    cfg = config_from_dict(d)
    pk = peaks()
    if args.fp32_check:
        print(json.dumps(fp32_check(cfg, args.model)))
        return 0
    if args.workload:
        print(json.dumps(run_long_context() if args.workload == "long-context" else run_workload(args.workload)))
        return 0
    model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0")

    prefill_ms = run_prefill(model, cfg)
    pf_flops = flops_prefill(cfg, PROMPT)
    launches0 = ops.launch_count()
    with ClockSampler() as clocks:
        tok_s, ms_step, bytes_step, key_range, phases = run_decode_point(model, cfg, BATCH, args.steps, args.warmup,
                                                                          with_phases=True)
    launches = ops.launch_count() - launches0
    points, points_frac = {}, {}
    if not args.skip_points:
        for name, batch in (("decode_b1", 1), ("decode_b64", 64)):
            point = run_decode_point(model, cfg, batch, args.steps, args.warmup)
            points[name] = point[0]
            # the same roofline as the headline's: used weights once and the live requests' cache, over the step's time
            points_frac[name] = round(point[2] / (point[1] / 1e3) / 1e9 / pk["hbm_gbs"], 4)
    e2e = run_e2e(model, cfg, args.steps, args.warmup)
    achieved = bytes_step / (ms_step / 1e3) / 1e9
    line = {
        "metric": f"decode tokens/s, Qwen3-{args.model.upper()} sizes, bf16, batch 8, 2048-token prompts, context 4096 "
                  f"(timed steps read {int(key_range[0])} to {int(key_range[1])} keys per sequence)",
        "value": tok_s, "unit": "tokens/s", "n_gpus": 1, "steps": min(args.steps, CONTEXT - PROMPT - args.warmup - 1),
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids",
        "impl": "ours",
        "config": {"model": f"Qwen3-{args.model.upper()} sizes", "layers": cfg.num_hidden_layers, "layers_of_config": full_layers,
                   "hidden_size": cfg.hidden_size, "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate_size": cfg.intermediate_size, "vocab_size": cfg.vocab_size,
                   "global_batch": BATCH, "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (15 GB of weights per step)", "peaks": pk["source"],
                   "keys_first_timed_step": int(key_range[0]), "keys_last_timed_step": int(key_range[1])},
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": {"value": PROMPT / (prefill_ms / 1e3), "tokens": PROMPT, "ms": prefill_ms,
                    "frac": pf_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "points_roofline_frac": points_frac,
        "phases": {"unit": "ms per decode step, kernel by kernel under the phase profiler (not the graph)",
                   **(phases or {})},
        "prefill_batched": {"tokens": BATCH * PROMPT, "ms": e2e["prefill_s"] * 1e3,
                            "value": BATCH * PROMPT / e2e["prefill_s"],
                            "frac_of_sustained": BATCH * pf_flops / e2e["prefill_s"] / (sustained_tflops() * 1e12),
                            "note": "the 8 prompts of the end-to-end run as one step, host work included; 0.2 s of dense "
                                    "products run under the power cap, so its fraction is taken against the sustained "
                                    "figure of the measured peaks, where the single prompt's 25 ms run at burst clocks"},
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
