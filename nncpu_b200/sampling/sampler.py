"""Choosing the next token of every live sequence of a step.

* greedy (temperature 0): the argmax kernel on the device; only token ids
  cross to the host (the reference fuses argmax into its output product for
  the same reason, crates/nncpu/src/model/forward.rs:989-1000);
* temperature without truncation: the sampling kernel on the device, which
  walks the distribution in token-id order (the reference walks it in rank
  order; the distribution is the same, the token drawn for a given uniform
  number is not);
* with top-k, top-p or min-p: the reference's chain on the host, in rank order.

Each sequence has a generator of its own, seeded ``seed + index``, so what a
sequence draws does not depend on which other sequences share its batch; a
single sequence with index 0 draws what the reference draws for that seed.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

from ..kernels import ops
from .chain import sample_from_logits
from .params import SamplerParams
from .rng import Mt19937_64


class Sampler:
    def __init__(self, params: SamplerParams, seed: int, vocab_size: int):
        params.check("sample")
        self.params = params
        self.seed = seed
        self.vocab_size = vocab_size
        self._rngs: Dict[int, Mt19937_64] = {}

    def rng(self, index: int) -> Mt19937_64:
        r = self._rngs.get(index)
        if r is None:
            r = self._rngs[index] = Mt19937_64(self.seed + index)
        return r

    def choose(self, logits: torch.Tensor, indices: Sequence[int]) -> List[int]:
        """``logits`` float32 [n, vocab] on the device, row i belonging to the
        sequence with index ``indices[i]``.  Returns one token id per row."""
        n = logits.shape[0]
        p = self.params
        if p.is_greedy:
            out = torch.empty(n, dtype=torch.int32, device=logits.device)
            ops.argmax(logits, out)
            return out.tolist()
        if not p.truncates(self.vocab_size):
            u = torch.tensor([self.rng(i).uniform(1.0) for i in indices], dtype=torch.float64).pin_memory()
            u = u.to(logits.device, non_blocking=True)
            out = torch.empty(n, dtype=torch.int32, device=logits.device)
            ops.sample_temperature(logits, u, out, p.temperature)
            return out.tolist()
        host = logits.to("cpu").numpy()
        return [sample_from_logits(host[r], p, self.rng(i)) for r, i in enumerate(indices)]
