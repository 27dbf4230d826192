"""The Python entry point, in the reference's manner
(crates/nncpu/src/lib.rs:131-271, crates/nncpu/src/session/engine.rs:95-352):

    model = Model.load("folder", dtype="bfloat16")
    session = Session(model, SessionParams(n_ctx=4096, seed=1, max_batch=8))
    results = session.generate([[1, 2, 3], [4, 5]], GenerateParams(max_tokens=32))

A ``Session`` owns an engine (model + cache).  Where the reference's session
holds one sequence, this one holds up to ``max_batch`` at a time; the
one-sequence calls ``eval`` / ``logits`` / ``sample`` / ``chat`` / ``reset``
keep the reference's meaning on a sequence of the session's own, whose cache
stays between calls.

With a tokenizer (``Session(model, params, tokenizer=...)``) pieces carry text
in whole UTF-8 characters beside the token id
(crates/nncpu/src/session/chat.rs:63-118), and ``chat`` adds a message to the
session's conversation as a ChatML turn and generates the reply
(crates/nncpu/src/session/engine.rs:316-328).
"""
from __future__ import annotations

import os
import threading
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch

from .cache import PAGE
from .engine.generate import generate as _generate, generate_on_slot as _generate_on_slot
from .engine.step import Engine
from .errors import ContextFull, InvalidArgument, NncpuError
from .sampling import GenerateParams, GenerateResult, Sampler, SamplerParams
from .text import TextStream, chat_turn, end_token_ids


@dataclass(frozen=True)
class SessionParams:
    """``n_ctx`` 0 = min(4096, the model's position range)
    (crates/nncpu/src/session/engine.rs:113-117); ``seed`` 0 = random
    (crates/nncpu/src/session/engine.rs:125); ``kv_f32`` keeps the cache in
    float32 whatever the run's element type (the reference's ``--kv-f32``);
    ``max_batch``: sequences generated together; ``system_prompt`` opens the
    session's conversation (crates/nncpu/src/session/mod.rs:37-83);
    ``reply_open`` is text the chat template puts at the start of every reply
    (Qwen3 without reasoning: ``"<think>\\n\\n</think>\\n\\n"``,
    crates/nncpu/src/tokenizer/mod.rs:994-997)."""
    n_ctx: int = 0
    seed: int = 0
    kv_f32: bool = False
    max_batch: int = 8
    system_prompt: str = ""
    reply_open: str = ""
    run_ahead: bool = True      # launch each decode step on the device's own choices before the host reads them


@dataclass(frozen=True)
class Piece:
    """One generated token of sequence ``index``, handed to ``on_piece``.  In a
    session with a tokenizer ``text`` holds the whole characters that this
    token completed (empty while a character is still cut off); when a sequence
    ends with bytes left over, a last piece with ``token`` None carries them."""
    index: int
    token: Optional[int]
    text: str = ""


class CancelHandle:
    """Asks the running call to stop at the next token boundary; usable from
    any thread (crates/nncpu/src/session/mod.rs:179-190)."""

    def __init__(self):
        self._flag = threading.Event()

    def cancel(self) -> None:
        self._flag.set()

    def _start_call(self) -> None:
        self._flag.clear()  # every call starts uncancelled

    def _is_set(self) -> bool:
        return self._flag.is_set()


class Session:
    _make_sampler = staticmethod(Sampler)    # (SamplerParams, seed, vocabulary size) -> chooser

    def __init__(self, model, params: SessionParams = SessionParams(), tokenizer=None, engine=None):
        """``engine``: an engine made elsewhere for ``model`` (tests pass a scripted one); by default the
        session makes its own, with room for ``max_batch`` sequences of ``n_ctx`` tokens and one more for the
        session's own sequence."""
        if params.n_ctx < 0 or params.max_batch < 1:
            raise InvalidArgument(f"n_ctx {params.n_ctx}, max_batch {params.max_batch}")
        self.model = model
        self.params = params
        self.tokenizer = tokenizer
        self.n_ctx = params.n_ctx if params.n_ctx > 0 else min(4096, model.spec.max_positions)
        per_seq = (self.n_ctx + PAGE - 1) // PAGE * PAGE
        self.engine = engine if engine is not None else Engine(
            model, max_tokens=per_seq * (params.max_batch + 1), max_seq_len=self.n_ctx,
            kv_dtype=torch.float32 if params.kv_f32 else None)
        self.seed = params.seed if params.seed != 0 else int.from_bytes(os.urandom(8), "little") | 1
        self._cancel = CancelHandle()
        self._own_slot: Optional[int] = None
        self._own_tokens: List[int] = []     # the session's own sequence: what the cache holds, then what waits
        self._own_logits: Optional[torch.Tensor] = None
        self._own_rngs: Optional[Sampler] = None
        self._n_generate_calls = 0

    # -- batches of requests -----------------------------------------------------

    def generate(self, prompts: Sequence[Sequence[int]], params: GenerateParams = GenerateParams(),
                 on_piece: Optional[Callable[[Piece], bool]] = None,
                 stop_token_ids: Optional[Sequence[int]] = None) -> List[GenerateResult]:
        """A continuation for every prompt (lists of token ids).  Sequences of
        a batch are prefilled in one step and decoded together; requests beyond
        ``max_batch`` run as later batches on the slots the earlier ones gave
        back.  ``on_piece(Piece)`` may return False to stop that sequence.
        ``stop_token_ids`` defaults to the configuration's end-of-sequence ids."""
        params.sampler.check("generate")
        if params.max_tokens < 0:
            raise InvalidArgument(f"generate: max_tokens {params.max_tokens}")
        stops = self._stops(stop_token_ids)
        sampler = self._make_sampler(params.sampler, self.seed + 1000003 * self._n_generate_calls, self.model.spec.vocab_size)
        self._n_generate_calls += 1
        self._cancel._start_call()
        on_token, on_finish = self._piece_callbacks(on_piece)
        # one slot's worth of pages is kept for the one-sequence calls
        return _generate(self.engine, sampler, prompts, params, stops, on_token, self._cancel._is_set,
                         max_batch=self.params.max_batch, n_ctx=self.n_ctx,
                         n_pages=self.engine.n_pages - (self.n_ctx + PAGE - 1) // PAGE, on_finish=on_finish,
                         run_ahead=self.params.run_ahead)

    def _stops(self, stop_token_ids):
        """The configuration's end-of-sequence ids and, with a tokenizer, the end markers its vocabulary
        holds (crates/nncpu/src/tokenizer/mod.rs:385-405); a caller's own list replaces both."""
        if stop_token_ids is not None:
            return stop_token_ids
        stops = list(self.model.spec.stop_token_ids)
        if self.tokenizer is not None:
            stops += [t for t in end_token_ids(self.tokenizer) if t not in stops]
        return stops

    def _piece_callbacks(self, on_piece):
        """``on_token`` and ``on_finish`` for the generation loop: pieces with text in whole characters when the
        session has a tokenizer, token ids alone otherwise."""
        if on_piece is None:
            return None, None
        tok = self.tokenizer
        if tok is None:
            return (lambda i, t: on_piece(Piece(i, t))), None
        streams = {}

        def on_token(i, t):
            stream = streams.get(i)
            if stream is None:
                stream = streams[i] = TextStream()
            return on_piece(Piece(i, t, stream.write(tok.token_bytes(t))))

        def on_finish(i):
            stream = streams.pop(i, None)
            rest = stream.finish() if stream is not None else ""
            if rest:
                on_piece(Piece(i, None, rest))
        return on_token, on_finish

    def cancel_handle(self) -> CancelHandle:
        return self._cancel

    # -- one sequence, step by step -------------------------------------------------

    def eval(self, tokens: Sequence[int]) -> None:
        """Runs ``tokens`` through the model after what this session's own
        sequence already holds (crates/nncpu/src/session/engine.rs:217-251)."""
        if len(tokens) == 0 and self.n_past() == len(self._own_tokens):
            return
        if self._own_slot is None:
            self._own_slot = self.engine.alloc_slot()
        waiting = self._own_tokens[self.n_past():] + [int(t) for t in tokens]
        # a copy: a one-token step returns a view of its decode graph's buffer, which the next step of that
        # size (this session's generate() included) overwrites
        held = self.n_past()
        try:
            self._own_logits = self.engine.step([self._own_slot], [waiting]).clone()
            self.engine.check_status()
        except BaseException:
            # the sequence stays what it was before the call (crates/nncpu/src/session/engine.rs:370-374)
            self._own_logits = None
            try:
                if self.engine.cache.length(self._own_slot) > held:
                    self.engine.cache.truncate(self._own_slot, held)
            except NncpuError:
                self.reset()        # a window or a state that cannot go back: the sequence starts over
            raise
        self._own_tokens += [int(t) for t in tokens]

    def logits(self) -> torch.Tensor:
        """float32 [vocab] on the device: the prediction after the last
        evaluated token (crates/nncpu/src/session/engine.rs:255-270)."""
        if self._own_logits is None:
            raise InvalidArgument("there is nothing to predict from: the context is empty")
        return self._own_logits[0]

    def sample(self, params: SamplerParams = SamplerParams()) -> int:
        """A next token for this session's own sequence; it is not evaluated
        (crates/nncpu/src/session/engine.rs:273-278)."""
        if self._own_logits is None:
            raise InvalidArgument("there is nothing to predict from: the context is empty")
        if self._own_rngs is None or self._own_rngs.params != params:
            old = self._own_rngs
            self._own_rngs = Sampler(params, self.seed, self.model.spec.vocab_size)
            if old is not None:
                self._own_rngs._rngs = old._rngs
        return self._own_rngs.choose(self._own_logits, [0])[0]

    def n_past(self) -> int:
        """Tokens of the session's own sequence that the cache holds."""
        return 0 if self._own_slot is None else min(self.engine.cache.length(self._own_slot), len(self._own_tokens))

    def tokens(self) -> List[int]:
        """The session's own sequence: evaluated tokens, then those that wait (a reply's last token)."""
        return list(self._own_tokens)

    def extend(self, tokens: Sequence[int], params: GenerateParams = GenerateParams(),
               on_piece: Optional[Callable[[Piece], bool]] = None,
               stop_token_ids: Optional[Sequence[int]] = None) -> GenerateResult:
        """Adds ``tokens`` to the session's own sequence and generates after
        them, as the reference's one-sequence ``generate`` does
        (crates/nncpu/src/session/engine.rs:289-299,598-690): the cache of
        earlier calls is kept, only what is new is evaluated, and the generated
        tokens (a stop token included) join the sequence; the last of them
        waits to be evaluated by the next call."""
        params.sampler.check("generate")
        if params.max_tokens < 0:
            raise InvalidArgument(f"generate: max_tokens {params.max_tokens}")
        context = self._own_tokens + [int(t) for t in tokens]
        if not context:
            raise InvalidArgument("there is nothing to continue: the context and the new tokens are both empty")
        if len(context) + 1 > self.n_ctx:
            # refused before anything changes (crates/nncpu/src/session/engine.rs:605-615)
            raise ContextFull(f"{len(context)} tokens of context ({len(tokens)} of them new) and room for one more "
                              f"do not fit the {self.n_ctx}-token context")
        if self._own_slot is None:
            self._own_slot = self.engine.alloc_slot()
        n_held = self.n_past()
        if n_held == len(context):
            # everything is evaluated already (eval() then extend([])): run the last token again from one back
            self.engine.cache.truncate(self._own_slot, n_held - 1)
            n_held -= 1
        elif self.engine.cache.length(self._own_slot) > n_held:
            self.engine.cache.truncate(self._own_slot, n_held)
        sampler = self._make_sampler(params.sampler, self.seed + 1000003 * self._n_generate_calls, self.model.spec.vocab_size)
        self._n_generate_calls += 1
        self._cancel._start_call()
        self._own_logits = None
        on_token, on_finish = self._piece_callbacks(on_piece)
        self._own_tokens = context
        return _generate_on_slot(self.engine, sampler, self._own_slot, self._own_tokens, n_held, params,
                                 self._stops(stop_token_ids), on_token, self._cancel._is_set, self.n_ctx, on_finish)

    def chat(self, message: str, params: GenerateParams = GenerateParams(),
             on_piece: Optional[Callable[[Piece], bool]] = None) -> GenerateResult:
        """One chat turn: ``message`` joins the session's conversation as a user
        turn in ChatML (the previous reply is closed first; the system prompt
        opens the first turn) and the reply is generated.  ``ContextFull``
        means that the turn does not fit; ``reset()`` makes room
        (crates/nncpu/src/session/engine.rs:300-328)."""
        if self.tokenizer is None:
            raise InvalidArgument("chat needs a tokenizer: Session(model, params, tokenizer=...)")
        end = self.tokenizer.special_id("<|im_end|>")
        closed = bool(self._own_tokens) and self._own_tokens[-1] == end
        turn = chat_turn(self.tokenizer, message, not self._own_tokens, closed, self.params.system_prompt,
                         self.params.reply_open)
        return self.extend(turn, params, on_piece)

    def reset(self) -> None:
        """Forgets this session's own sequence (crates/nncpu/src/session/engine.rs:201-209)."""
        if self._own_slot is not None:
            self.engine.free_slot(self._own_slot)
        self._own_slot = None
        self._own_tokens = []
        self._own_logits = None
