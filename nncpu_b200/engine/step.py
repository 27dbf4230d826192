"""The step function: one batch of sequences, each bringing its next tokens.

A step runs only the tokens it is given, as one flat batch, against the cache
that earlier steps left, appends their keys and values, and returns the logits
at the wanted places.  Sequences of a batch start together with prompts of
unequal lengths (one step), then go on by one token each; a step may also mix
lengths freely, because every kernel works from per-token (sequence, position)
pairs.  Arguments are checked before anything changes, as the reference does
for its one-sequence forward pass (crates/nncpu/src/model/forward.rs:851-886).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import perf
from ..cache import Cache, pages_for
from ..errors import InvalidArgument, translating_oom
from ..kernels import ops
from ..parts import EntryCache
from ..parts.runtime import Arena


@dataclass
class StepContext:
    """What kernels and parts see of a step.  Device tensors are int32."""
    n_tokens: int
    n_seqs: int
    n_wanted: int
    tok_ids: torch.Tensor       # [n_tokens] token ids
    tok_seq: torch.Tensor       # [n_tokens] index of the token's sequence in this step (-1: padding)
    tok_pos: torch.Tensor       # [n_tokens] position in its sequence
    seq_slots: torch.Tensor     # [n_seqs] cache slot of each sequence
    cu_seqlens: torch.Tensor    # [n_seqs + 1] first flat token of each sequence
    logit_rows: torch.Tensor    # [n_wanted] flat tokens whose logits are wanted
    block_tables: List[torch.Tensor]  # per cache group: [n_seqs, width] page ids
    q_lens: List[int]           # host: tokens per sequence in this step
    kv_lens: List[int]          # host: length of each sequence after this step
    is_decode: bool             # every sequence brings exactly one token
    h2d_bytes: int = 0          # bytes of metadata copied to the device for this step
    max_kv_len: int = 0         # host: an upper bound of the longest sequence after this step
    memo: Dict = field(default_factory=dict)  # per-step results shared between layers
    next_norm: Optional[object] = None    # a NormRequest for the part that is running: see parts.base.NormRequest
    after_block: Optional[object] = None  # the request of the block that follows, for the running block's last part

    def span_sum(self, window: int = 0) -> int:
        """Keys that the step's tokens attend to, summed over the tokens: a token at position p sees p + 1
        keys, or the last ``window`` of them."""
        key = ("span_sum", window)
        n = self.memo.get(key)
        if n is None:
            n = 0
            for q, after in zip(self.q_lens, self.kv_lens):
                first = after - q + 1                      # keys seen by the sequence's first new token
                if window > 0:
                    n += sum(min(first + i, window) for i in range(q))
                else:
                    n += q * first + q * (q - 1) // 2
            self.memo[key] = n
        return n

    def entry_cache(self, cache: Cache, entry: int) -> EntryCache:
        g = cache.group_of(entry)
        if g is None:
            return EntryCache(None, None, None, False, cache.state(entry))
        k, v = cache.kv(entry)
        return EntryCache(k, v, self.block_tables[g], cache.owns_kv(entry), cache.state(entry))


class Staging:
    """A ring of pinned host buffers for the metadata of steps: a buffer is
    reused only after the copy that read it has finished."""

    def __init__(self, n: int = 4):
        self.bufs: List[Optional[torch.Tensor]] = [None] * n
        self.events: List[Optional[torch.cuda.Event]] = [None] * n
        self.turn = 0

    def take(self, n_ints: int) -> Tuple[torch.Tensor, int]:
        i = self.turn = (self.turn + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.bufs[i]
        if buf is None or buf.numel() < n_ints:
            buf = self.bufs[i] = torch.empty(max(n_ints, 4096), dtype=torch.int32).pin_memory()
        return buf[:n_ints], i

    def sent(self, i: int) -> None:
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


def make_context(cache: Cache, slots: Sequence[int], tokens: Sequence[Sequence[int]],
                 want: Sequence[Sequence[int]], staging: Optional[Staging] = None, alloc=None) -> StepContext:
    """The step's metadata as one block of int32, copied to the device once.
    Call after ``cache.prepare``: the page tables must already cover the new tokens.
    ``alloc(n, dtype=...)`` gives the device block (the step's arena); without it the allocator does."""
    starts = [cache.length(s) for s in slots]
    q_lens = [len(t) for t in tokens]
    n, B = sum(q_lens), len(slots)
    cu = np.zeros(B + 1, dtype=np.int64)
    np.cumsum(q_lens, out=cu[1:])
    rows = [int(cu[b]) + i for b in range(B) for i in want[b]]
    tables = [cache.block_table(g, slots) for g in range(len(cache.groups))]
    offsets = [0, n, 2 * n, 3 * n, 3 * n + B, 3 * n + 2 * B + 1]
    total = offsets[5] + len(rows)
    table_at = []
    for t in tables:
        table_at.append(total)
        total += B * len(t[0])
    on_gpu = cache.device.type == "cuda"
    if staging is not None and on_gpu:
        host, turn = staging.take(total)
    else:
        host = torch.empty(total, dtype=torch.int32)
        if on_gpu:
            host = host.pin_memory()
    a = host.numpy()
    if n:
        a[0:n] = np.concatenate([np.asarray(t, dtype=np.int64) for t in tokens if len(t)])
        a[n:2 * n] = np.repeat(np.arange(B), q_lens)
        a[2 * n:3 * n] = np.arange(n) - np.repeat(cu[:-1] - np.asarray(starts, dtype=np.int64), q_lens)
    a[offsets[3]:offsets[4]] = slots
    a[offsets[4]:offsets[5]] = cu
    a[offsets[5]:offsets[5] + len(rows)] = rows
    for at, t in zip(table_at, tables):
        a[at:at + B * len(t[0])] = np.asarray(t, dtype=np.int64).reshape(-1)
    if alloc is not None and on_gpu:
        dev = alloc(total, dtype=torch.int32)
        dev.copy_(host, non_blocking=True)
    else:
        dev = host.to(cache.device, non_blocking=True)
    if staging is not None and on_gpu:
        staging.sent(turn)
    views = [dev[offsets[i]:offsets[i + 1]] for i in range(5)] + [dev[offsets[5]:offsets[5] + len(rows)]]
    bts = [dev[at:at + B * len(t[0])].view(B, len(t[0])) for at, t in zip(table_at, tables)]
    return StepContext(n_tokens=n, n_seqs=B, n_wanted=len(rows), tok_ids=views[0], tok_seq=views[1],
                       tok_pos=views[2], seq_slots=views[3], cu_seqlens=views[4], logit_rows=views[5],
                       block_tables=bts, q_lens=q_lens, kv_lens=[s + q for s, q in zip(starts, q_lens)],
                       is_decode=all(q == 1 for q in q_lens), h2d_bytes=total * 4,
                       max_kv_len=max(s + q for s, q in zip(starts, q_lens)))


def shape_context(cache: Cache, n_tokens: int, n_seqs: int, n_wanted: int, max_kv_len: int) -> StepContext:
    """A step of these sizes without data: every tensor is shape-only (``meta``).  For the pass that measures
    how much memory a step needs."""
    def ints(*shape):
        return torch.empty(shape, dtype=torch.int32, device="meta")
    width = max(1, pages_for(max_kv_len))
    per = max(1, n_tokens // n_seqs)
    q_lens = [per] * (n_seqs - 1) + [n_tokens - per * (n_seqs - 1)]
    return StepContext(n_tokens=n_tokens, n_seqs=n_seqs, n_wanted=n_wanted, tok_ids=ints(n_tokens), tok_seq=ints(n_tokens),
                       tok_pos=ints(n_tokens), seq_slots=ints(n_seqs), cu_seqlens=ints(n_seqs + 1),
                       logit_rows=ints(n_wanted), block_tables=[ints(n_seqs, width) for _ in cache.groups],
                       q_lens=q_lens, kv_lens=list(q_lens), is_decode=all(q == 1 for q in q_lens),
                       max_kv_len=max_kv_len)


class Engine:
    """A model with its cache.  ``step`` is the only way tokens reach the model.

    A step's intermediate tensors come out of one arena that is sized when the engine is made, by a pass of the
    model's forward over the shapes of the largest expected step (``max_step_tokens`` tokens, by default the
    cache's capacity up to 8 192): a step asks the allocator for nothing.  A step that turns out larger (more
    tokens, or many rows of logits wanted) is served by the allocator once, and the arena is as large from then on
    (the reference sizes its scratch once, crates/nncpu/src/model/kv.rs:295-332)."""

    def __init__(self, model, max_tokens: int, n_slots: Optional[int] = None, max_seq_len: Optional[int] = None,
                 kv_dtype: Optional[torch.dtype] = None, use_graphs: bool = True,
                 max_step_tokens: Optional[int] = None):
        from .decode_graph import PROMPT_GRAPH_MAX, DecodeGraphs
        self._prompt_graph_max = PROMPT_GRAPH_MAX
        self.model = model
        self.graphs = DecodeGraphs(self) if use_graphs else None
        self._last_graph = None   # the graph of the last step, if that step ran through one
        self._staging = Staging()
        self.h2d_bytes_last_step = 0
        requests, cache_of = model.cache_requests()
        rt = model.rt
        # A sequence may grow as long as the cache lets it.  The model's own position range only sets a
        # session's default context, as in the reference (crates/nncpu/src/session/engine.rs:113-117): rotary
        # positions need no table, so nothing breaks beyond it.
        self.cache = Cache(requests, cache_of, max_tokens, kv_dtype or rt.dtype, rt.device, n_slots=n_slots,
                           max_seq_len=max_seq_len)
        self.vocab_size = model.spec.vocab_size
        self.arena = Arena(rt.device)
        self.max_step_tokens = min(max_step_tokens or 8192, self.cache.max_tokens)
        self._size_arena()

    def _size_arena(self) -> None:
        """Runs the forward pass over shapes alone for a prompt step of ``max_step_tokens`` tokens (one sequence,
        and as many sequences as fit) and makes the arena hold the larger of the two."""
        rt, n = self.model.rt, self.max_step_tokens
        self.arena.measuring = True
        try:
            with rt.using(self.arena), ops.shapes_only():
                for n_seqs in {1, max(1, min(n, self.cache.n_slots, 256))}:
                    self.arena.begin()
                    ctx = shape_context(self.cache, n, n_seqs, n_seqs, min(n, self.cache.max_seq_len))
                    rt.empty(3 * n + 4 * n_seqs + 1 + sum(t.numel() for t in ctx.block_tables), dtype=torch.int32)
                    self.model.forward(ctx, self.cache)
        except Exception:
            self.arena.peak = 0      # a part that cannot run on shapes alone: the arena learns from the first steps
        finally:
            self.arena.measuring = False
        with translating_oom(f"the arena of a step of {n} tokens ({self.arena.peak / 2 ** 20:.0f} MiB)"):
            self.arena.begin()

    @property
    def max_seq_len(self) -> int:
        return self.cache.max_seq_len

    @property
    def n_pages(self) -> int:
        return self.cache.n_pages

    # -- slots -----------------------------------------------------------------

    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    # -- the step ----------------------------------------------------------------

    def check(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
              want: Sequence[Sequence[int]]) -> None:
        if not slots or len(slots) != len(tokens) or len(want) != len(tokens):
            raise InvalidArgument(f"a step of {len(slots)} slots, {len(tokens)} token lists and {len(want)} want lists")
        for b, (toks, w) in enumerate(zip(tokens, want)):
            if len(toks) == 0:
                raise InvalidArgument(f"sequence {b} brings no token to the step")
            for t in toks:
                if not 0 <= t < self.vocab_size:
                    raise InvalidArgument(f"token {t} is outside the vocabulary [0, {self.vocab_size})")
            for i in w:
                if not 0 <= i < len(toks):
                    raise InvalidArgument(f"sequence {b}: wanted place {i} is outside its {len(toks)} tokens")

    def build_context(self, slots, tokens, want) -> StepContext:
        ctx = make_context(self.cache, slots, tokens, want, self._staging, alloc=self.model.rt.empty)
        self.h2d_bytes_last_step = ctx.h2d_bytes
        return ctx

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """Feeds ``tokens[b]`` to the sequence in ``slots[b]``.  ``want[b]``
        lists the places among ``tokens[b]`` whose logits are returned
        (default: the last).  Returns float32 [n_wanted, vocab] on the device,
        rows in the order of the sequences and of ``want``; None if nothing is
        wanted.  The result lives in the step's arena (or its graph's buffer):
        it is valid until the engine's next step, so copy what must last longer
        (the reference's logits are likewise those of the last evaluation,
        crates/nncpu/src/session/engine.rs:255-270)."""
        if want is None:
            want = [[len(t) - 1] for t in tokens]
        slots = [int(s) for s in slots]
        self.check(slots, tokens, want)
        self.cache.prepare(slots, [len(t) for t in tokens])
        if (self.graphs is not None and not perf.enabled() and all(len(t) == 1 for t in tokens)
                and all(list(w) == [0] for w in want)):
            try:
                with translating_oom(f"a decode step of {len(slots)} sequences"):
                    g = self.graphs.get(len(slots))
                    logits = g.run(slots, [t[0] for t in tokens])
            except BaseException:
                self.cache.rollback(slots)
                raise
            self.h2d_bytes_last_step = g.h2d_bytes
            self.cache.commit(slots, [1] * len(slots))
            self._last_graph = g
            return logits
        self._last_graph = None
        if (self.graphs is not None and not perf.enabled() and len(slots) == 1
                and 1 < len(tokens[0]) <= self._prompt_graph_max and list(want[0]) == [len(tokens[0]) - 1]
                and not self.cache.has_state):
            # one sequence's short prompt (a chat turn): one captured launch instead of a host-bound string of them
            try:
                with translating_oom(f"a prompt step of {len(tokens[0])} tokens"):
                    g = self.graphs.prompt(len(tokens[0]))
                    logits = g.run(slots[0], tokens[0])
            except BaseException:
                self.cache.rollback(slots)
                raise
            self.h2d_bytes_last_step = g.h2d_bytes
            self.cache.commit(slots, [len(tokens[0])])
            return logits
        try:
            with translating_oom(f"a step of {sum(len(t) for t in tokens)} tokens in {len(slots)} sequences"), \
                    self.model.rt.using(self.arena):
                self.arena.begin()
                ctx = self.build_context(slots, tokens, want)
                logits = self.model.forward(ctx, self.cache)
        except BaseException:
            self.cache.rollback(slots)     # the step did not happen: the cache is as it was
            raise
        self.cache.commit(slots, ctx.q_lens)
        return logits

    # -- decoding without a host round trip per step -----------------------------

    def choice_buffer(self, n: int) -> Optional[torch.Tensor]:
        """Where the last graph step's choices live on the device: int32 [n],
        filled by the graph itself with the greedy choice of every sequence; a
        chooser that draws on the device overwrites it.  None if the last step
        did not run through a graph."""
        g = self._last_graph
        return None if g is None else g.next_ids[:n]

    def fetch_choices(self, n: int):
        """Starts the copy of the choice buffer to pinned host memory, in
        stream order.  Returns ``(event, ids)``: after ``event.synchronize()``
        ``ids[:n]`` holds the tokens.  None if the last step did not run through a graph."""
        g = self._last_graph
        if g is None:
            return None
        self.model.rt.post_status()     # the status word travels with the tokens: checking it costs no wait
        return g.fetch_ids(n)

    def check_status(self) -> None:
        """Raises ``ExtensionError`` if a kernel of an earlier step gave up a bounded wait.  Call where the
        device has been waited for."""
        self.model.rt.check_status()

    def step_again(self, slots: Sequence[int]) -> torch.Tensor:
        """One more decode step for exactly the sequences of the last graph
        step, each fed its token from the choice buffer, which never leaves
        the device."""
        slots = [int(s) for s in slots]
        g = self._last_graph
        if g is None or g.slots != tuple(slots):
            raise InvalidArgument("step_again needs the sequences of the last decode step, in its order")
        n = len(slots)
        self.cache.prepare(slots, [1] * n)
        logits = g.run(slots, None)
        self.h2d_bytes_last_step = g.h2d_bytes
        self.cache.commit(slots, [1] * n)
        return logits

    def decode_run(self, slots: Sequence[int], first_tokens, n_steps: int) -> torch.Tensor:
        """``n_steps`` greedy decode steps for the sequences in ``slots``
        without a stop check: the first step feeds ``first_tokens`` (a list, or
        an int32 device tensor), every later step feeds the previous step's
        choice, which stays on the device.  Returns the chosen tokens, int32
        [n_steps, len(slots)] on the device."""
        slots = [int(s) for s in slots]
        n = len(slots)
        out = torch.empty((n_steps, n), dtype=torch.int32, device=self.cache.device)
        if self.graphs is None:
            raise InvalidArgument("decode_run replays captured steps: the engine was made with use_graphs=False")
        graphs = self.graphs
        g = graphs.get(n)
        for i in range(n_steps):
            self.cache.prepare(slots, [1] * n)
            if i == 0:
                if isinstance(first_tokens, torch.Tensor):
                    g.next_ids[:n].copy_(first_tokens.to(torch.int32))
                    g.run(slots, None)
                else:
                    g.run(slots, [int(t) for t in first_tokens])
            else:
                g.run(slots, None)
            self.cache.commit(slots, [1] * n)
            out[i].copy_(g.next_ids[:n])
        return out
