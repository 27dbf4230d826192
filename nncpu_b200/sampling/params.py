"""How the next token is chosen and how a reply is generated: the reference's
``SamplerParams``, ``GenerateParams``, ``StopReason`` and ``GenerateResult``
(crates/nncpu/src/session/mod.rs:86-177) with the same names, meanings and
defaults."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum
from typing import List

from ..errors import InvalidArgument


@dataclass(frozen=True)
class SamplerParams:
    """top-k, then top-p, then min-p on the model's own distribution, then
    temperature over what survives.  ``temperature`` 0 = greedy; ``top_k`` 0 =
    all; ``top_p`` 1 = off; ``min_p`` 0 = off."""
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05

    @staticmethod
    def greedy() -> "SamplerParams":
        return SamplerParams(temperature=0.0)

    def check(self, function: str = "sample") -> None:
        """crates/nncpu/src/session/mod.rs:122-131."""
        def unit(v):
            return isinstance(v, (int, float)) and math.isfinite(v) and 0.0 <= v <= 1.0
        ok = (isinstance(self.temperature, (int, float)) and math.isfinite(self.temperature)
              and self.temperature >= 0 and unit(self.top_p) and unit(self.min_p)
              and isinstance(self.top_k, int) and self.top_k >= 0)
        if not ok:
            raise InvalidArgument(f"{function}: temperature must be >= 0, top_k >= 0, and top_p/min_p in [0, 1]")

    @property
    def is_greedy(self) -> bool:
        return self.temperature <= 0.0

    def truncates(self, vocab: int) -> bool:
        """Whether any of top-k, top-p, min-p removes candidates."""
        return (0 < self.top_k < vocab) or (0.0 < self.top_p < 1.0) or self.min_p > 0.0


@dataclass(frozen=True)
class GenerateParams:
    """``max_tokens`` 0 = until a stop token or a full context."""
    max_tokens: int = 0
    sampler: SamplerParams = field(default_factory=SamplerParams)


class StopReason(Enum):
    END_OF_TURN = "EndOfTurn"      # the model produced a stop token
    MAX_TOKENS = "MaxTokens"       # max_tokens were generated
    CONTEXT_FULL = "ContextFull"   # the sequence reached the context size
    CALLBACK = "Callback"          # the callback returned False
    CANCELLED = "Cancelled"        # cancel() was called


@dataclass
class GenerateResult:
    """What one sequence's generation did.  ``tokens`` are the generated
    tokens, the stop token not among them; ``n_generated == len(tokens)``."""
    stop: StopReason = StopReason.END_OF_TURN
    n_prompt: int = 0
    n_generated: int = 0
    prefill: float = 0.0   # seconds spent on the prompt (shared by a batch)
    decode: float = 0.0    # seconds spent generating (shared by a batch)
    tokens: List[int] = field(default_factory=list)
