"""The generation loop: batches of prompts of unequal lengths, one prefill
step, then one token per live sequence and step until every sequence stopped.

The decisions per sampled token are the reference's, in its order
(crates/nncpu/src/session/engine.rs:476-506): a stop token ends the sequence
and is neither counted nor streamed; otherwise the token is counted and
streamed; the callback may stop the sequence; a full context stops it; then
``max_tokens``.  A cancel is seen before each sampling round
(crates/nncpu/src/session/engine.rs:657-660).  The last generated token is
never run through the model (crates/nncpu/src/session/engine.rs:665-667).

A sequence that stops leaves the batch: later steps carry only the live ones,
and its slot and pages go back to the cache at once.  Requests beyond
``max_batch`` wait for the next batch; batches run one after another and never
take on new members.

The loop talks to an engine through ``alloc_slot``, ``free_slot``, ``step``
and ``max_seq_len`` only, and to a chooser through ``choose(logits, indices)``,
so its decisions can be tested with scripted stand-ins for both.

Decoding does not wait for the host where the choice can be made on the
device: when the chooser says so (``chooses_on_device``; greedy choices are
even made by the engine's decode graph itself, ``greedy_on_device``) and the
engine offers ``choice_buffer``, ``fetch_choices`` and ``step_again``, the
chooser's kernels write the tokens into the engine's buffer, the next step is
launched on top of them, and the host reads the tokens meanwhile and takes its
decisions one step behind.  A sequence that the host then stops has run one
step too many, which nobody sees: its slot is freed.  Steps in which a count
limit (context, ``max_tokens``) can end a sequence are not run ahead.

Wherever the loop has waited for the device it asks the engine whether a
kernel gave up a bounded wait (``check_status``, if the engine has it): a step
whose kernel did not finish its work raises instead of handing out tokens, and
the batch's slots are freed on the way out.
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional, Sequence

from ..cache import PAGE, pages_for
from ..errors import ContextFull, InvalidArgument
from ..sampling.params import GenerateParams, GenerateResult, StopReason


def plan_batches(prompt_lens: Sequence[int], max_new: Sequence[int], max_batch: int, n_pages: int) -> List[List[int]]:
    """Cuts request indices 0..n-1, in order, into batches of at most
    ``max_batch`` whose prompts plus room to generate fit ``n_pages`` pages."""
    batches, cur, used = [], [], 0
    for i, (p, g) in enumerate(zip(prompt_lens, max_new)):
        need = pages_for(p + g)
        if need > n_pages:
            raise ContextFull(f"request {i}: {p} prompt tokens and room for {g} more need {need} cache pages "
                              f"of {PAGE} tokens, the cache has {n_pages}")
        if cur and (len(cur) >= max_batch or used + need > n_pages):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def generate(engine, chooser, prompts: Sequence[Sequence[int]], params: GenerateParams,
             stop_token_ids: Sequence[int] = (), on_token: Optional[Callable[[int, int], bool]] = None,
             cancelled: Callable[[], bool] = lambda: False, max_batch: int = 64,
             n_ctx: Optional[int] = None, n_pages: Optional[int] = None,
             on_finish: Optional[Callable[[int], None]] = None, run_ahead: bool = True) -> List[GenerateResult]:
    """Generates a continuation for every prompt.  ``chooser.choose(logits,
    indices)`` picks one token per logits row; ``on_token(index, token)`` is
    called for every generated token and may return False to stop that
    sequence; ``on_finish(index)`` is called once when a sequence has stopped.
    ``run_ahead`` False keeps every step behind the host's decisions (the
    tokens are the same either way).  Results come in the order of the prompts."""
    n_ctx = n_ctx or engine.max_seq_len
    stops = frozenset(int(t) for t in stop_token_ids)
    if not prompts:
        return []
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise InvalidArgument(f"prompt {i} is empty: there is nothing to continue")
        # the prompt plus at least one generated token must fit (crates/nncpu/src/session/engine.rs:605-615)
        if len(p) + 1 > n_ctx:
            raise ContextFull(f"prompt {i} of {len(p)} tokens does not fit the {n_ctx}-token context")
    room = [min(n_ctx - len(p), params.max_tokens) if params.max_tokens > 0 else n_ctx - len(p) for p in prompts]
    batches = plan_batches([len(p) for p in prompts], room, max_batch,
                           n_pages if n_pages is not None else engine.n_pages)
    results: List[Optional[GenerateResult]] = [None] * len(prompts)
    for batch in batches:
        _run_batch(engine, chooser, [(i, list(prompts[i])) for i in batch], params, stops, on_token, cancelled,
                   n_ctx, results, on_finish, run_ahead=run_ahead)
    return results  # type: ignore[return-value]


def generate_on_slot(engine, chooser, slot: int, tokens: List[int], n_evaluated: int, params: GenerateParams,
                     stop_token_ids: Sequence[int] = (), on_token: Optional[Callable[[int, int], bool]] = None,
                     cancelled: Callable[[], bool] = lambda: False, n_ctx: Optional[int] = None,
                     on_finish: Optional[Callable[[int], None]] = None) -> GenerateResult:
    """Continues the one sequence that lives in ``slot``: ``tokens`` is its whole
    context, of which the cache already holds the first ``n_evaluated``; the rest
    is run as one step, then tokens are generated as in ``generate``.  The slot
    stays with the caller, and ``tokens`` is extended in place with what was
    generated (a stop token included), as the reference keeps its context
    (crates/nncpu/src/session/engine.rs:476-481,598-690)."""
    n_ctx = n_ctx or engine.max_seq_len
    if n_evaluated >= len(tokens):
        raise InvalidArgument("there is nothing to continue from: no token is waiting to be evaluated")
    if len(tokens) + 1 > n_ctx:
        raise ContextFull(f"{len(tokens)} tokens of context leave no room in the {n_ctx}-token context")
    results: List[Optional[GenerateResult]] = [None]
    _run_batch(engine, chooser, [(0, tokens)], params, frozenset(int(t) for t in stop_token_ids), on_token, cancelled,
               n_ctx, results, on_finish, held={0: (slot, n_evaluated)})
    return results[0]  # type: ignore[return-value]


def _run_batch(engine, chooser, members, params, stops, on_token, cancelled, n_ctx, results, on_finish=None,
               held=None, run_ahead=True) -> None:
    """``held``: index -> (slot, tokens already in the cache) for sequences that continue on a slot of the
    caller's, which is not given back."""
    held = held or {}
    check_status = getattr(engine, "check_status", None) or (lambda: None)
    live = []  # [index, slot, tokens so far (prompt + generated), result]
    on_device = (run_ahead
                 and (getattr(chooser, "chooses_on_device", False) or getattr(chooser, "greedy_on_device", False))
                 and all(hasattr(engine, a) for a in ("choice_buffer", "fetch_choices", "step_again")))

    def settle(rows, chosen):
        """Takes one chosen token per sequence of ``rows``; returns the sequences that go on."""
        still = []
        for (idx, slot, toks, r), tok in zip(rows, chosen):
            tok = int(tok)
            toks.append(tok)
            if tok in stops:
                r.stop = StopReason.END_OF_TURN
            else:
                r.n_generated += 1
                r.tokens.append(tok)
                if on_token is not None and on_token(idx, tok) is False:
                    r.stop = StopReason.CALLBACK
                elif len(toks) >= n_ctx:
                    r.stop = StopReason.CONTEXT_FULL
                elif params.max_tokens > 0 and r.n_generated >= params.max_tokens:
                    r.stop = StopReason.MAX_TOKENS
                else:
                    still.append([idx, slot, toks, r])
                    continue
            if idx not in held:
                engine.free_slot(slot)
            if on_finish is not None:
                on_finish(idx)
        return still

    try:
        first = []
        for idx, prompt in members:
            slot, start = held[idx] if idx in held else (engine.alloc_slot(), 0)
            live.append([idx, slot, prompt, GenerateResult(n_prompt=len(prompt) - start)])
            first.append(prompt[start:])
        t0 = time.perf_counter()
        logits = engine.step([s for _, s, _, _ in live], first)
        done_results = [r for _, _, _, r in live]
        prefill = None
        t1 = t0
        while live:
            if cancelled():
                for idx, _, _, r in live:
                    r.stop = StopReason.CANCELLED
                    if on_finish is not None:
                        on_finish(idx)
                break
            ahead = None
            buffer = engine.choice_buffer(len(live)) if on_device and prefill is not None else None
            if buffer is not None:
                # The tokens of the step in flight are chosen on the device (a greedy choice is there already,
                # made by the step itself): start their copy to the host and, unless a count limit may end a
                # sequence with this very token, launch the next step on top of them.
                if not getattr(chooser, "greedy_on_device", False):
                    chooser.enqueue(logits, [idx for idx, _, _, _ in live], buffer)
                event, ids = engine.fetch_choices(len(live))
                if all(len(toks) + 2 <= n_ctx and (params.max_tokens <= 0 or r.n_generated + 2 <= params.max_tokens)
                       for _, _, toks, r in live):
                    ahead = engine.step_again([s for _, s, _, _ in live])
                event.synchronize()
                chosen = ids[:len(live)].tolist()
            else:
                chosen = chooser.choose(logits, [idx for idx, _, _, _ in live])
            check_status()      # the device has been waited for: did every kernel of the step finish its work?
            if prefill is None:  # the first choice waits for the prompt step to finish
                t1 = time.perf_counter()
                prefill = t1 - t0
            still = settle(live, chosen)
            if ahead is not None and len(still) == len(live):
                live, logits = still, ahead     # nobody stopped: the step run ahead is the step in flight
                continue
            if ahead is not None and still:
                # Somebody stopped, so the step run ahead carried sequences that are gone; for the others it is
                # their next step all the same.  Its choices are read by row and settled like any others; the
                # next round starts with a plain step.
                going_on = {m[0] for m in still}
                rows = [k for k, m in enumerate(live) if m[0] in going_on]
                if not getattr(chooser, "greedy_on_device", False):
                    chooser.enqueue(ahead, [m[0] for m in live], engine.choice_buffer(len(live)))
                event, ids = engine.fetch_choices(len(live))
                event.synchronize()
                check_status()
                still = settle(still, [int(ids[k]) for k in rows])
            live = still
            if live:
                logits = engine.step([s for _, s, _, _ in live], [[t[-1]] for _, _, t, _ in live])
        t2 = time.perf_counter()
        for r in done_results:
            r.prefill = prefill if prefill is not None else t2 - t0
            r.decode = t2 - t1
        for (idx, _), r in zip(members, done_results):
            results[idx] = r
    finally:
        for idx, slot, _, _ in live:
            if idx not in held:
                engine.free_slot(slot)
