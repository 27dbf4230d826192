"""Choosing the next token of every live sequence of a step.

* greedy (temperature 0): the argmax kernel on the device; only token ids
  cross to the host (the reference fuses argmax into its output product for
  the same reason, crates/nncpu/src/model/forward.rs:989-1000);
* temperature without truncation: the sampling kernel on the device, which
  walks the distribution in token-id order (the reference walks it in rank
  order; the distribution is the same, the token drawn for a given uniform
  number is not);
* with top-k (the default, 40): the top-k kernel picks the candidates on the
  device and the host runs the rest of the reference's chain on those few;
* with top-p or min-p but no top-k: the best 1024 candidates and the row's
  softmax denominator come from the device; the host runs the chain on them and
  reads the whole row only if neither cut falls among them.

Each sequence has a generator of its own, seeded ``seed + index``, so what a
sequence draws does not depend on which other sequences share its batch; a
single sequence with index 0 draws what the reference draws for that seed.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

from ..kernels import ops
from .chain import sample_from_candidates, sample_from_logits
from .params import SamplerParams
from .rng import Mt19937_64


_NO_TOPK_CANDIDATES = 1024


class Sampler:
    def __init__(self, params: SamplerParams, seed: int, vocab_size: int):
        params.check("sample")
        self.params = params
        self.seed = seed
        self.vocab_size = vocab_size
        self._rngs: Dict[int, Mt19937_64] = {}

    @property
    def greedy_on_device(self) -> bool:
        """Greedy choices are the first largest logit, which the engine's decode graph computes itself."""
        return self.params.is_greedy

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
        if 0 < p.top_k < self.vocab_size and p.top_k <= 1024:
            # the device picks the k candidates; only they cross to the host, which runs the rest of the chain
            vals = torch.empty(n, p.top_k, dtype=torch.float32, device=logits.device)
            ids = torch.empty(n, p.top_k, dtype=torch.int32, device=logits.device)
            ops.topk(logits, vals, ids)
            vals, ids = vals.cpu().numpy(), ids.cpu().numpy()
            return [sample_from_candidates(vals[r], ids[r], p, self.rng(i)) for r, i in enumerate(indices)]
        if self.vocab_size > 4 * _NO_TOPK_CANDIDATES:
            # no top-k: top-p and min-p nearly always cut among the best few, so fetch those and the
            # row's denominator, and fall back to the whole row only where the cut lies further out
            vals = torch.empty(n, _NO_TOPK_CANDIDATES, dtype=torch.float32, device=logits.device)
            ids = torch.empty(n, _NO_TOPK_CANDIDATES, dtype=torch.int32, device=logits.device)
            total = torch.empty(n, dtype=torch.float64, device=logits.device)
            ops.topk(logits, vals, ids)
            ops.row_exp_sum(logits, total)
            vals, ids, total = vals.cpu().numpy(), ids.cpu().numpy(), total.cpu().numpy()
            out = []
            for r, i in enumerate(indices):
                rng = self.rng(i)
                t = sample_from_candidates(vals[r], ids[r], p, rng, whole_total=float(total[r]))
                if t is None:
                    t = sample_from_logits(logits[r].cpu().numpy(), p, rng)
                out.append(t)
            return out
        host = logits.to("cpu").numpy()
        return [sample_from_logits(host[r], p, self.rng(i)) for r, i in enumerate(indices)]
