"""The reference's sampling chain on one row of logits, on the host:
top-k, top-p and min-p on the distribution at temperature 1, then temperature
over the survivors and one uniform draw in rank order (higher logit first,
then lower id); NaN counts as -inf and is never drawn
(crates/nncpu/src/session/sample.rs:69-88,121-201).
"""
from __future__ import annotations

from typing import Optional

import numpy as np

from .params import SamplerParams
from .rng import Mt19937_64


def argmax_first(logits: np.ndarray) -> int:
    """The first largest value; NaN never wins (crates/nncpu/src/model/forward.rs:1003-1011)."""
    x = np.where(np.isnan(logits), -np.inf, logits)
    return int(np.argmax(x))


def sample_from_logits(logits: np.ndarray, p: SamplerParams, rng: Mt19937_64) -> int:
    """One draw from a whole row of logits."""
    logits = np.asarray(logits, dtype=np.float32)
    n = logits.shape[0]
    l = np.where(np.isnan(logits), np.float32(-np.inf), logits)
    ids = np.arange(n)
    k = p.top_k if 0 < p.top_k < n else n
    if k < n:
        # the k best by (logit desc, id asc): everything above the k-th value, then the lowest ids at it
        kth = np.partition(l, n - k)[n - k]
        above = np.nonzero(l > kth)[0]
        ties = np.nonzero(l == kth)[0][:k - above.size]
        keep = np.concatenate([above, ties])
        return sample_from_candidates(l[keep], keep, p, rng)
    return sample_from_candidates(l, ids, p, rng)


def sample_from_candidates(values: np.ndarray, ids: np.ndarray, p: SamplerParams, rng: Mt19937_64,
                           whole_total: Optional[float] = None) -> Optional[int]:
    """One draw from the candidates that top-k left (any order; NaN already -inf): ranking, top-p,
    min-p, temperature, draw.

    With ``whole_total`` the candidates are only the best of a longer row that has no top-k:
    ``whole_total`` is that row's sum of exp(logit - largest).  The result is the whole row's if top-p
    or min-p cuts inside the candidates; if neither does, None."""
    values = np.asarray(values, dtype=np.float32)
    ids = np.asarray(ids)
    rank = np.lexsort((ids, -values))
    order = ids[rank]
    cand_l = values[rank]
    if cand_l.size == 0 or not np.isfinite(cand_l[0]):
        return int(order[0]) if order.size else 0
    top = cand_l[0]
    prob = np.exp((cand_l - top).astype(np.float32)).astype(np.float32)
    total = float(prob.astype(np.float64).sum()) if whole_total is None else float(whole_total)
    keep = cand_l.size
    cut_inside = whole_total is None
    if 0.0 < p.top_p < 1.0:
        cum = np.cumsum(prob.astype(np.float64) / total)
        hit = np.nonzero(cum >= float(np.float32(p.top_p)))[0]
        if hit.size:
            keep = int(hit[0]) + 1
            cut_inside = True
    if p.min_p > 0.0:
        floor = np.float32(p.min_p) * prob[0]
        i = 1
        while i < keep and prob[i] >= floor:
            i += 1
        cut_inside = cut_inside or i < keep
        keep = i
    if not cut_inside:
        return None
    inv_t = 1.0 / float(np.float32(p.temperature))
    pt = np.exp((cand_l[:keep] - top).astype(np.float32).astype(np.float64) * inv_t).astype(np.float32)
    r = rng.uniform(float(pt.astype(np.float64).sum()))
    for w, i in zip(pt, order[:keep]):
        r -= float(w)
        if r <= 0.0:
            return int(i)
    return int(order[keep - 1])
