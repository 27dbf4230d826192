"""Decode steps, and the short prompt steps of one sequence, as CUDA graphs.

A decode step is launch-bound when run kernel by kernel: a few hundred small
launches per token.  For every batch size (rounded up to a power of two) the
engine captures the step once over static buffers and replays it afterwards;
per step the host only refreshes a small block of int32 metadata (positions,
page tables) and copies it to the device.

Rows beyond the live sequences are padding: their sequence index and their
slot are -1, so no kernel writes the cache for them, their outputs are zeros,
and a part that keeps per-sequence state reads and writes the spare last row
of its state area (index -1), which no sequence owns.

The step that captures a graph runs the model once, kernel by kernel, and
returns that result; the captured graph is replayed from the next step of that
size on.  A part whose step is not idempotent (per-sequence state) therefore
advances exactly once per step.
"""
from __future__ import annotations

import gc
import weakref
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import perf
from ..cache import pages_for
from ..kernels import ops
from ..parts.runtime import Arena
from .step import StepContext

_RING = 4  # pinned host copies of the metadata in flight


def bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class DecodeGraph:
    """Static buffers and the captured step for one padded batch size."""

    def __init__(self, engine, size: int):
        self._engine, self.size = weakref.ref(engine), size  # no cycle: graphs die with their engine
        cache = engine.cache
        dev = cache.device
        self.width = pages_for(cache.max_seq_len)
        n_groups = len(cache.groups)
        B = size
        # layout of the metadata block (int32): tok_seq, tok_pos, seq_slots, cu_seqlens, logit_rows, page tables
        self.o_seq, self.o_pos, self.o_slot, self.o_cu = 0, B, 2 * B, 3 * B
        self.o_rows = 4 * B + 1
        self.o_tables = [5 * B + 1 + g * B * self.width for g in range(n_groups)]
        self.n_meta = 5 * B + 1 + n_groups * B * self.width
        self.meta = torch.zeros(self.n_meta, dtype=torch.int32, device=dev)
        self.tok_ids = torch.zeros(B, dtype=torch.int32, device=dev)
        self.next_ids = torch.zeros(B, dtype=torch.int32, device=dev)
        self.host = [torch.zeros(self.n_meta, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.host_np = [h.numpy() for h in self.host]
        self.events: List[Optional[torch.cuda.Event]] = [None] * _RING
        self.turn = 0
        self.tok_host = [torch.zeros(B, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        m = self.meta
        self.ctx = StepContext(
            n_tokens=B, n_seqs=B, n_wanted=B, tok_ids=self.tok_ids, tok_seq=m[self.o_seq:self.o_seq + B],
            tok_pos=m[self.o_pos:self.o_pos + B], seq_slots=m[self.o_slot:self.o_slot + B],
            cu_seqlens=m[self.o_cu:self.o_cu + B + 1], logit_rows=m[self.o_rows:self.o_rows + B],
            block_tables=[m[o:o + B * self.width].view(B, self.width) for o in self.o_tables],
            q_lens=[1] * B, kv_lens=[0] * B, is_decode=True, max_kv_len=cache.max_seq_len)
        self.logits: Optional[torch.Tensor] = None
        self.arena = Arena(dev)     # the captured step's intermediate tensors: its addresses are part of the graph
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.n_kernels = 0
        self.slots: Optional[tuple] = None
        self.gens: Optional[tuple] = None
        self.pages_seen: List[List[int]] = []
        self.h2d_bytes = 0

    @property
    def engine(self):
        return self._engine()

    def _fill(self, slots: Sequence[int], tokens: Optional[Sequence[int]]) -> None:
        """Writes this step's metadata into the next pinned copy and sends it."""
        cache, B, n = self.engine.cache, self.size, len(slots)
        i = self.turn = (self.turn + 1) % _RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        a = self.host_np[i]
        prev = self.host_np[(i - 1) % _RING]
        # the tables of the step before may be built upon only if these are the same sequences in the same slots
        gens = tuple(cache.generation[s] for s in slots)
        same = self.slots == tuple(slots) and self.gens == gens
        if same:
            a[:] = prev
        else:
            a[:] = -1
            a[self.o_seq:self.o_seq + n] = np.arange(n)
            a[self.o_pos:self.o_pos + B] = 0
            a[self.o_slot:self.o_slot + n] = slots       # padding rows keep slot -1
            a[self.o_cu:self.o_cu + B + 1] = np.arange(B + 1)
            a[self.o_rows:self.o_rows + n] = np.arange(n)
            self.slots = tuple(slots)
            self.gens = gens
            self.pages_seen = [[0] * n for _ in cache.groups]
        a[self.o_pos:self.o_pos + n] = [cache.lengths[s] for s in slots]
        for g, group in enumerate(cache.groups):
            seen = self.pages_seen[g]
            windowed = group.request.window > 0
            for b, s in enumerate(slots):
                table = group.tables[s]
                if windowed or len(table) != seen[b]:
                    o = self.o_tables[g] + b * self.width
                    a[o:o + len(table)] = table
                    seen[b] = len(table)
        self.meta.copy_(self.host[i], non_blocking=True)
        self.h2d_bytes = self.n_meta * 4
        if tokens is not None:
            th = self.tok_host[i]
            th[:n] = torch.as_tensor(tokens, dtype=torch.int32)
            th[n:] = 0
            self.tok_ids.copy_(th, non_blocking=True)
            self.h2d_bytes += B * 4
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev

    def fetch_ids(self, n: int):
        """Copies the greedy choices of the step just launched to pinned memory, in stream order (so before a
        later step overwrites them).  Returns (event, int32 host tensor)."""
        i = self.fetch_turn = (getattr(self, "fetch_turn", -1) + 1) % _RING
        if not hasattr(self, "ids_host"):
            self.ids_host = [torch.empty(self.size, dtype=torch.int32).pin_memory() for _ in range(_RING)]
            self.ids_events = [torch.cuda.Event() for _ in range(_RING)]
        self.ids_host[i][:n].copy_(self.next_ids[:n], non_blocking=True)
        self.ids_events[i].record()
        return self.ids_events[i], self.ids_host[i]

    def _forward(self) -> None:
        with self.engine.model.rt.using(self.arena):
            self.arena.begin()
            self.logits = self.engine.model.forward(self.ctx, self.engine.cache)
        ops.argmax(self.logits, self.next_ids)

    def run(self, slots: Sequence[int], tokens: Optional[Sequence[int]]) -> torch.Tensor:
        """One decode step for ``slots``.  ``tokens`` None: the step's tokens
        are the previous step's greedy choices, which never left the device.
        Returns float32 logits [len(slots), vocab], valid until the next step."""
        with perf.paused():      # events cannot be timed inside a graph: a replay is not attributed to phases
            return self._run(slots, tokens)

    def _run(self, slots, tokens):
        self.ctx.memo.clear()
        self._fill(slots, tokens)
        if tokens is None:
            self.tok_ids.copy_(self.next_ids, non_blocking=True)
        if self.graph is None:
            # The first step of this size runs kernel by kernel and its result is the step's result.  The same
            # work is then captured, not run: a second run would advance per-sequence state twice.
            self._forward()
            eager = self.logits
            self.arena.begin()          # now as large as that run needed;
            self.arena.frozen = True    # from here on its addresses belong to the graph
            before = ops.launch_count()
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            self.ctx.memo.clear()
            # Nothing may free device memory or destroy another graph while the stream captures:
            # collect garbage now and keep the collector off until the capture has ended.
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    self._forward()
            finally:
                if gc_was_on:
                    gc.enable()
            self.n_kernels = ops.launch_count() - before
            ops.add_launches(-self.n_kernels)  # capturing launches nothing
            self.graph = g
            self.logits.copy_(eager)  # the graph's own buffer holds this step's logits until its first replay
        else:
            self.graph.replay()
            ops.add_launches(self.n_kernels)
        return self.logits[:len(slots)]


PROMPT_GRAPH_MIN = 16     # the smallest padded size of a captured prompt step
PROMPT_GRAPH_MAX = 256    # longer prompts keep the device busy about as long as the host needs to launch them (measured at
#                           the 8B sizes, a layer: 17 tokens 223 -> 142 us, 64: 197 -> 153, 128: 217 -> 179, 256: 255 -> 233;
#                           300 tokens padded to 512 would take 311 us against 301 launched kernel by kernel)


class PromptGraph:
    """Static buffers and the captured step of ONE sequence that brings up to ``size`` new tokens and wants the
    logits of its last one: the step that a chat turn, or a single short prompt, begins with.  Launched kernel by
    kernel from Python such a step of a few dozen tokens is bound by the host (some 17 us a launch); captured for
    its padded size (a power of two from 16 to 256) it is one launch.  The tokens beyond the prompt's own are padding: they belong to
    no sequence (index -1), so nothing is written to the cache for them, attention leaves them out, and what the
    products compute in their rows is never read."""

    def __init__(self, engine, size: int):
        self._engine, self.size = weakref.ref(engine), size
        cache = engine.cache
        dev = cache.device
        self.width = pages_for(cache.max_seq_len)
        n_groups = len(cache.groups)
        T = size
        # layout of the metadata block (int32): tok_seq, tok_pos, the slot, cu_seqlens, the wanted row, page tables
        self.o_seq, self.o_pos, self.o_slot, self.o_cu, self.o_row = 0, T, 2 * T, 2 * T + 1, 2 * T + 3
        self.o_tables = [2 * T + 4 + g * self.width for g in range(n_groups)]
        self.n_meta = 2 * T + 4 + n_groups * self.width
        self.meta = torch.zeros(self.n_meta, dtype=torch.int32, device=dev)
        self.tok_ids = torch.zeros(T, dtype=torch.int32, device=dev)
        self.host = [torch.zeros(self.n_meta, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.host_np = [h.numpy() for h in self.host]
        self.tok_host = [torch.zeros(T, dtype=torch.int32).pin_memory() for _ in range(_RING)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * _RING
        self.turn = 0
        m = self.meta
        self.ctx = StepContext(
            n_tokens=T, n_seqs=1, n_wanted=1, tok_ids=self.tok_ids, tok_seq=m[self.o_seq:self.o_seq + T],
            tok_pos=m[self.o_pos:self.o_pos + T], seq_slots=m[self.o_slot:self.o_slot + 1],
            cu_seqlens=m[self.o_cu:self.o_cu + 2], logit_rows=m[self.o_row:self.o_row + 1],
            block_tables=[m[o:o + self.width].view(1, self.width) for o in self.o_tables],
            q_lens=[T], kv_lens=[T], is_decode=False, max_kv_len=cache.max_seq_len)
        self.logits: Optional[torch.Tensor] = None
        self.arena = Arena(dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.n_kernels = 0
        self.h2d_bytes = 0

    @property
    def engine(self):
        return self._engine()

    def _fill(self, slot: int, tokens: Sequence[int]) -> None:
        cache, T, n = self.engine.cache, self.size, len(tokens)
        i = self.turn = (self.turn + 1) % _RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        a = self.host_np[i]
        start = cache.lengths[slot]
        a[:] = -1
        a[self.o_seq:self.o_seq + n] = 0
        a[self.o_pos:self.o_pos + T] = 0
        a[self.o_pos:self.o_pos + n] = np.arange(start, start + n)
        a[self.o_slot] = slot
        a[self.o_cu:self.o_cu + 2] = (0, n)
        a[self.o_row] = n - 1
        for g, group in enumerate(cache.groups):
            table = group.tables[slot]
            a[self.o_tables[g]:self.o_tables[g] + len(table)] = table
        self.meta.copy_(self.host[i], non_blocking=True)
        th = self.tok_host[i]
        th[:n] = torch.as_tensor(tokens, dtype=torch.int32)
        th[n:] = 0
        self.tok_ids.copy_(th, non_blocking=True)
        self.h2d_bytes = (self.n_meta + T) * 4
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev

    def _forward(self) -> None:
        with self.engine.model.rt.using(self.arena):
            self.arena.begin()
            self.logits = self.engine.model.forward(self.ctx, self.engine.cache)

    def run(self, slot: int, tokens: Sequence[int]) -> torch.Tensor:
        """The step: ``tokens`` appended to the sequence in ``slot``.  Returns float32 logits [1, vocab] of the last
        token, valid until the next step."""
        with perf.paused():
            self.ctx.memo.clear()
            self._fill(slot, tokens)
            if self.graph is None:
                # as for decode steps: the first step of this size runs kernel by kernel and is the step's result;
                # the same work is then captured, not run
                self._forward()
                eager = self.logits
                self.arena.begin()
                self.arena.frozen = True
                before = ops.launch_count()
                g = torch.cuda.CUDAGraph()
                torch.cuda.synchronize()
                self.ctx.memo.clear()
                gc.collect()
                gc_was_on = gc.isenabled()
                gc.disable()
                try:
                    with torch.cuda.graph(g, capture_error_mode="thread_local"):
                        self._forward()
                finally:
                    if gc_was_on:
                        gc.enable()
                self.n_kernels = ops.launch_count() - before
                ops.add_launches(-self.n_kernels)
                self.graph = g
                self.logits.copy_(eager)
            else:
                self.graph.replay()
                ops.add_launches(self.n_kernels)
            return self.logits


class DecodeGraphs:
    def __init__(self, engine):
        self._engine = weakref.ref(engine)
        self.by_size: Dict[int, DecodeGraph] = {}
        self.prompts: Dict[int, PromptGraph] = {}

    def get(self, n: int) -> DecodeGraph:
        size = bucket(n)
        g = self.by_size.get(size)
        if g is None:
            g = self.by_size[size] = DecodeGraph(self._engine(), size)
        return g

    def prompt(self, n: int) -> PromptGraph:
        """The captured step of one sequence with ``n`` new tokens (2 <= n <= PROMPT_GRAPH_MAX)."""
        size = max(PROMPT_GRAPH_MIN, bucket(n))
        g = self.prompts.get(size)
        if g is None:
            g = self.prompts[size] = PromptGraph(self._engine(), size)
        return g
