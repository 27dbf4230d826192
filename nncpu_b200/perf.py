"""The phase profiler: where a step's time goes, phase by phase.

After the reference's profiler (crates/nncpu/src/perf.rs): named slots, a scope
that adds its time and the bytes it streamed to a slot, ``perf_enable`` /
``perf_reset`` / ``perf_report`` (crates/nncpu/src/lib.rs:59), and a table of
ms, %, calls, us/call and effective bandwidth (crates/nncpu/src/perf.rs:156-218).
Off by default, and free when off.  Process-wide, so meant for one session at a
time.

What differs, because the work runs on a GPU: a scope brackets its kernels with
a pair of CUDA events on the current stream and the times are read when a
report is asked for, so the host never waits inside a step; a scope also takes
the multiply-adds of its phase, and the table shows TFLOP/s beside GB/s and,
when the device's measured peaks are given, the larger of the two as a fraction
of its peak.  CUDA events cannot be timed inside a captured graph: while the
profiler is on, decode steps run kernel by kernel instead of replaying their
graph, which the report's first line says; a replay that is asked for
explicitly (``Engine.decode_run``, ``Engine.step_again``) is not attributed.

Byte and flop model, as the reference's (crates/nncpu/src/model/mod.rs:391-398,
crates/nncpu/src/model/forward.rs:382-386): a matrix phase streams its weights
once; attention streams, for every token, the keys and values of its span;
norms, rotation, activation and embedding count no bytes.

A part of another architecture names its own slot: ``scope("moe_route")``
creates it on first use, after the known ones.
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional, Tuple

# the reference's slot names for the phases this architecture has, in forward order, plus the token choice
SLOTS = ("embed", "norm", "attn_qkv", "attn_rope", "attn_core", "attn_out", "ffn_gate_up", "ffn_act", "ffn_down",
         "lm_head", "sample")

_on = False
_paused = 0
_lock = threading.Lock()
_totals: Dict[str, List[float]] = {}        # slot -> [ns, bytes, flops, calls]
_pending: List[Tuple[str, object, object, float, float]] = []
_first = None                               # start event of the first scope since the last reset
_span_ns = 0.0                              # from there to the end of the last scope read so far
_event_pool: List[object] = []
_MAX_PENDING = 8192


class _NullScope:
    __slots__ = ()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NULL = _NullScope()


class _Scope:
    __slots__ = ("slot", "bytes", "flops", "start")

    def __init__(self, slot: str, nbytes: float, flops: float):
        self.slot, self.bytes, self.flops, self.start = slot, nbytes, flops, None

    def __enter__(self):
        global _first
        self.start = _event()
        self.start.record()
        if _first is None:
            _first = self.start
        return self

    def __exit__(self, *exc):
        end = _event()
        end.record()
        with _lock:
            _pending.append((self.slot, self.start, end, self.bytes, self.flops))
            drain = len(_pending) >= _MAX_PENDING
        if drain:
            _drain()
        return False


def _event():
    import torch
    with _lock:
        if _event_pool:
            return _event_pool.pop()
    return torch.cuda.Event(enable_timing=True)


def _drain() -> None:
    """Waits for the device and turns the finished event pairs into totals."""
    with _lock:
        todo, _pending[:] = list(_pending), []
    if not todo:
        return
    import torch
    global _span_ns
    torch.cuda.synchronize()
    for slot, a, b, nbytes, flops in todo:
        add(slot, a.elapsed_time(b) * 1e6, nbytes, flops)
    if _first is not None:
        _span_ns = max(_span_ns, _first.elapsed_time(todo[-1][2]) * 1e6)
    with _lock:
        for _, a, b, _, _ in todo:
            if len(_event_pool) < 2 * _MAX_PENDING and a is not _first:
                _event_pool.extend((a, b))


def enabled() -> bool:
    """Whether scopes record right now (on, and not paused around a graph replay)."""
    return _on and _paused == 0


def scope(slot: str, nbytes: float = 0, flops: float = 0):
    """``with scope("attn_qkv", nbytes=..., flops=...):`` around the launches of a phase."""
    if not (_on and _paused == 0):
        return _NULL
    return _Scope(slot, nbytes, flops)


class paused:
    """Scopes inside record nothing: around work that cannot be timed with events (a captured graph)."""

    def __enter__(self):
        global _paused
        _paused += 1

    def __exit__(self, *exc):
        global _paused
        _paused -= 1
        return False


def add(slot: str, ns: float, nbytes: float = 0, flops: float = 0) -> None:
    """Adds one call of ``ns`` nanoseconds to ``slot`` (crates/nncpu/src/perf.rs:104-109)."""
    with _lock:
        t = _totals.setdefault(slot, [0.0, 0.0, 0.0, 0])
        t[0] += ns
        t[1] += nbytes
        t[2] += flops
        t[3] += 1


def perf_enable(enabled: bool = True) -> None:
    """Turns the process-wide phase profiler on or off.  While it is on, decode steps run kernel by kernel."""
    global _on
    if _on and not enabled:
        _drain()
    _on = bool(enabled)


def perf_reset() -> None:
    """Zeroes the profiler's totals; what is still in flight is dropped with them."""
    global _first, _span_ns
    _drain()
    with _lock:
        _totals.clear()
        _first, _span_ns = None, 0.0


def perf_span_ms() -> float:
    """Device time from the start of the first phase to the end of the last one since the last reset: what the
    phases' sum falls short of it went to the seams between them (and to the host, where the device waited)."""
    _drain()
    return _span_ns / 1e6


def perf_totals() -> Dict[str, dict]:
    """Per slot that was called: ms, calls, bytes, flops, in the report's order."""
    _drain()
    with _lock:
        names = [s for s in SLOTS if s in _totals] + [s for s in _totals if s not in SLOTS]
        return {s: {"ms": _totals[s][0] / 1e6, "calls": int(_totals[s][3]), "bytes": _totals[s][1],
                    "flops": _totals[s][2]} for s in names}


def perf_report(title: str = "", n_tokens: int = 0, peaks: Optional[dict] = None) -> str:
    """A table of time, bandwidth and arithmetic rate per phase since the last reset; ``n_tokens`` adds a
    per-token line when positive.  ``peaks`` ({"hbm_gbs": ..., "bf16_tflops": ...}, the device's measured copy
    bandwidth and matrix rate) adds each phase's fraction of the peak that bounds it."""
    totals = perf_totals()
    total_ns = sum(t["ms"] for t in totals.values()) * 1e6
    if total_ns == 0:
        return f"nncpu perf ({title}): no samples\n"
    out = [f"nncpu perf - {title} (timed with CUDA events; decode steps ran kernel by kernel)"]
    head = f"  {'phase':<12} {'ms':>10} {'%':>7} {'calls':>10} {'us/call':>10} {'GB/s':>10} {'TFLOP/s':>10}"
    rule = f"  {'-' * 12} {'-' * 10} {'-' * 7} {'-' * 10} {'-' * 10} {'-' * 10} {'-' * 10}"
    if peaks:
        head += f" {'of peak':>12}"
        rule += f" {'-' * 12}"
    out += [head, rule]
    total_bytes = 0.0
    for name, t in totals.items():
        ns = t["ms"] * 1e6
        line = (f"  {name:<12} {t['ms']:>10.1f} {100.0 * ns / total_ns:>6.1f}% {t['calls']:>10} "
                f"{ns / 1e3 / t['calls']:>10.1f}")
        gbs = t["bytes"] / ns if ns > 0 else 0.0
        tfs = t["flops"] / ns / 1e3 if ns > 0 else 0.0
        line += f" {gbs:>10.1f}" if t["bytes"] > 0 else f" {'':>10}"
        line += f" {tfs:>10.1f}" if t["flops"] > 0 else f" {'':>10}"
        if peaks and ns > 0 and (t["bytes"] > 0 or t["flops"] > 0):
            f_mem = gbs / peaks["hbm_gbs"] if peaks.get("hbm_gbs") else 0.0
            f_mma = tfs / peaks["bf16_tflops"] if peaks.get("bf16_tflops") else 0.0
            line += f" {max(f_mem, f_mma):>6.2f} {'hbm' if f_mem >= f_mma else 'mma':>5}"
        out.append(line.rstrip())
        total_bytes += t["bytes"]
    out.append(f"  {'TOTAL':<12} {total_ns / 1e6:>10.1f} {100.0:>6.1f}%")
    if _span_ns > 0:
        out.append(f"  the phases cover {100.0 * total_ns / _span_ns:.0f}% of the {_span_ns / 1e6:.1f} ms between the "
                   f"first and the last of them")
    if total_bytes > 0:
        out.append(f"  memory traffic: {total_bytes / 2 ** 30:.2f} GB @ {total_bytes / total_ns:.1f} GB/s effective")
    if n_tokens > 0:
        out.append(f"  {total_ns / 1e6 / n_tokens:.2f} ms/token over {n_tokens} tokens")
    return "\n".join(out) + "\n"
