"""Choosing the next token of every live sequence of a step.

* greedy (temperature 0): the argmax kernel on the device; only token ids
  cross to the host (the reference fuses argmax into its output product for
  the same reason, crates/nncpu/src/model/forward.rs:989-1000);
* temperature without truncation: the sampling kernel on the device, which
  walks the distribution in token-id order (the reference walks it in rank
  order; the distribution is the same, the token drawn for a given uniform
  number is not);
* with top-k up to 1024 (the default is 40): the whole chain runs on the
  device in one kernel: candidates by radix select, ranking by a bitonic
  sort, then top-p, min-p, temperature and the draw in rank order with the
  reference's arithmetic; the host only supplies each sequence's uniform
  number.  (A row without any finite logit is answered without a draw by the
  reference; here its uniform number is drawn and not used.)
* with top-p or min-p but no top-k: the best 1024 candidates and the row's
  softmax denominator come from the device; the host runs the chain on them and
  reads the whole row only if neither cut falls among them.

Each sequence has a generator of its own, seeded ``seed + index``, so what a
sequence draws does not depend on which other sequences share its batch; a
single sequence with index 0 draws what the reference draws for that seed.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .. import perf
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
        self._u_host: List[Optional[torch.Tensor]] = [None] * 4     # pinned staging for the uniform numbers
        self._u_events: List[Optional[torch.cuda.Event]] = [None] * 4
        self._u_turn = 0

    @property
    def greedy_on_device(self) -> bool:
        """Greedy choices are the first largest logit, which the engine's decode graph computes itself."""
        return self.params.is_greedy

    @property
    def chooses_on_device(self) -> bool:
        """Whether ``enqueue`` can make the choice with kernels alone, leaving the tokens on the device."""
        p = self.params
        return p.is_greedy or not p.truncates(self.vocab_size) or 0 < p.top_k <= min(1024, self.vocab_size - 1)

    def rng(self, index: int) -> Mt19937_64:
        r = self._rngs.get(index)
        if r is None:
            r = self._rngs[index] = Mt19937_64(self.seed + index)
        return r

    def _uniforms(self, indices: Sequence[int], device) -> torch.Tensor:
        """One uniform number in [0, 1) from each sequence's generator, on the device."""
        n = len(indices)
        i = self._u_turn = (self._u_turn + 1) % len(self._u_host)
        if self._u_events[i] is not None:
            self._u_events[i].synchronize()
        host = self._u_host[i]
        if host is None or host.numel() < n:
            host = self._u_host[i] = torch.empty(max(n, 64), dtype=torch.float64).pin_memory()
        host[:n] = torch.tensor([self.rng(j).uniform(1.0) for j in indices], dtype=torch.float64)
        dev = host[:n].to(device, non_blocking=True)
        ev = self._u_events[i] or torch.cuda.Event()
        ev.record()
        self._u_events[i] = ev
        return dev

    def enqueue(self, logits: torch.Tensor, indices: Sequence[int], out: torch.Tensor) -> None:
        """Launches the choice for every row of ``logits`` into ``out`` (int32 on the device) without waiting for
        it; only where ``chooses_on_device``."""
        p = self.params
        with perf.scope("sample"):
            if p.is_greedy:
                ops.argmax(logits, out)
            elif not p.truncates(self.vocab_size):
                ops.sample_temperature(logits, self._uniforms(indices, logits.device), out, p.temperature)
            else:
                ops.sample_chain(logits, self._uniforms(indices, logits.device), out, p.top_k, p.temperature, p.top_p,
                                 p.min_p)

    def choose(self, logits: torch.Tensor, indices: Sequence[int]) -> List[int]:
        """``logits`` float32 [n, vocab] on the device, row i belonging to the
        sequence with index ``indices[i]``.  Returns one token id per row."""
        n = logits.shape[0]
        p = self.params
        if self.chooses_on_device:
            out = torch.empty(n, dtype=torch.int32, device=logits.device)
            self.enqueue(logits, indices, out)
            return out.tolist()
        if not 0 < p.top_k < self.vocab_size and self.vocab_size > 4 * _NO_TOPK_CANDIDATES:
            # no top-k: top-p and min-p nearly always cut among the best few, so fetch those and the
            # row's denominator, and fall back to the whole row only where the cut lies further out
            vals = torch.empty(n, _NO_TOPK_CANDIDATES, dtype=torch.float32, device=logits.device)
            ids = torch.empty(n, _NO_TOPK_CANDIDATES, dtype=torch.int32, device=logits.device)
            total = torch.empty(n, dtype=torch.float64, device=logits.device)
            with perf.scope("sample"):
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
