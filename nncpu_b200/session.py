"""The Python entry point, in the reference's manner
(crates/nncpu/src/lib.rs:131-271, crates/nncpu/src/session/engine.rs:95-352):

    model = Model.load("folder", dtype="bfloat16")
    session = Session(model, SessionParams(n_ctx=4096, seed=1, max_batch=8))
    results = session.generate([[1, 2, 3], [4, 5]], GenerateParams(max_tokens=32))

A ``Session`` owns an engine (model + cache).  Where the reference's session
holds one sequence, this one holds up to ``max_batch`` at a time; the
one-sequence calls ``eval`` / ``logits`` / ``sample`` / ``reset`` keep the
reference's meaning on a sequence of their own.
"""
from __future__ import annotations

import os
import threading
import time
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch

from .cache import PAGE
from .engine.generate import generate as _generate
from .engine.step import Engine
from .errors import InvalidArgument
from .sampling import GenerateParams, GenerateResult, Sampler, SamplerParams


@dataclass(frozen=True)
class SessionParams:
    """``n_ctx`` 0 = min(4096, the model's position range)
    (crates/nncpu/src/session/engine.rs:113-117); ``seed`` 0 = random
    (crates/nncpu/src/session/engine.rs:125); ``kv_f32`` keeps the cache in
    float32 whatever the run's element type (the reference's ``--kv-f32``);
    ``max_batch``: sequences generated together."""
    n_ctx: int = 0
    seed: int = 0
    kv_f32: bool = False
    max_batch: int = 8


@dataclass(frozen=True)
class Piece:
    """One generated token of sequence ``index``, handed to ``on_piece``."""
    index: int
    token: int


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
    def __init__(self, model, params: SessionParams = SessionParams()):
        if params.n_ctx < 0 or params.max_batch < 1:
            raise InvalidArgument(f"n_ctx {params.n_ctx}, max_batch {params.max_batch}")
        self.model = model
        self.params = params
        self.n_ctx = params.n_ctx if params.n_ctx > 0 else min(4096, model.spec.max_positions)
        per_seq = (self.n_ctx + PAGE - 1) // PAGE * PAGE
        self.engine = Engine(model, max_tokens=per_seq * (params.max_batch + 1), max_seq_len=self.n_ctx,
                             kv_dtype=torch.float32 if params.kv_f32 else None)
        self.seed = params.seed if params.seed != 0 else int.from_bytes(os.urandom(8), "little") | 1
        self._cancel = CancelHandle()
        self._own_slot: Optional[int] = None
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
        stops = self.model.spec.stop_token_ids if stop_token_ids is None else stop_token_ids
        sampler = Sampler(params.sampler, self.seed + 1000003 * self._n_generate_calls, self.model.spec.vocab_size)
        self._n_generate_calls += 1
        self._cancel._start_call()
        on_token = None if on_piece is None else (lambda i, t: on_piece(Piece(i, t)))
        # one slot's worth of pages is kept for the one-sequence calls
        return _generate(self.engine, sampler, prompts, params, stops, on_token, self._cancel._is_set,
                         max_batch=self.params.max_batch, n_ctx=self.n_ctx,
                         n_pages=self.engine.n_pages - (self.n_ctx + PAGE - 1) // PAGE)

    def cancel_handle(self) -> CancelHandle:
        return self._cancel

    # -- one sequence, step by step -------------------------------------------------

    def eval(self, tokens: Sequence[int]) -> None:
        """Runs ``tokens`` through the model after what this session's own
        sequence already holds (crates/nncpu/src/session/engine.rs:217-251)."""
        if len(tokens) == 0:
            return
        if self._own_slot is None:
            self._own_slot = self.engine.alloc_slot()
        self._own_logits = self.engine.step([self._own_slot], [list(tokens)])

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
        return 0 if self._own_slot is None else self.engine.cache.length(self._own_slot)

    def reset(self) -> None:
        """Forgets this session's own sequence (crates/nncpu/src/session/engine.rs:201-209)."""
        if self._own_slot is not None:
            self.engine.free_slot(self._own_slot)
        self._own_slot = None
        self._own_logits = None
