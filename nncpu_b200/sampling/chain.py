"""The reference's sampling chain on one row of logits, on the host:
top-k, top-p and min-p on the distribution at temperature 1, then temperature
over the survivors and one uniform draw in rank order (higher logit first,
then lower id); NaN counts as -inf and is never drawn
(crates/nncpu/src/session/sample.rs:69-88,121-201).
"""
from __future__ import annotations

import numpy as np

from .params import SamplerParams
from .rng import Mt19937_64


def argmax_first(logits: np.ndarray) -> int:
    """The first largest value; NaN never wins (crates/nncpu/src/model/forward.rs:1003-1011)."""
    x = np.where(np.isnan(logits), -np.inf, logits)
    return int(np.argmax(x))


def sample_from_logits(logits: np.ndarray, p: SamplerParams, rng: Mt19937_64) -> int:
    logits = np.asarray(logits, dtype=np.float32)
    n = logits.shape[0]
    l = np.where(np.isnan(logits), np.float32(-np.inf), logits)
    ids = np.arange(n)
    k = p.top_k if 0 < p.top_k < n else n
    if k < n:
        # the k best by (logit desc, id asc): everything above the k-th value, then ties by id
        order = np.lexsort((ids, -l))[:k]
    else:
        order = np.lexsort((ids, -l))
    cand_l = l[order]
    if cand_l.size == 0 or not np.isfinite(cand_l[0]):
        return int(order[0]) if order.size else 0
    top = cand_l[0]
    prob = np.exp((cand_l - top).astype(np.float32)).astype(np.float32)
    total = float(prob.astype(np.float64).sum())
    keep = cand_l.size
    if 0.0 < p.top_p < 1.0:
        cum = np.cumsum(prob.astype(np.float64) / total)
        hit = np.nonzero(cum >= float(np.float32(p.top_p)))[0]
        if hit.size:
            keep = int(hit[0]) + 1
    if p.min_p > 0.0:
        floor = np.float32(p.min_p) * prob[0]
        i = 1
        while i < keep and prob[i] >= floor:
            i += 1
        keep = i
    inv_t = 1.0 / float(np.float32(p.temperature))
    pt = np.exp((cand_l[:keep] - top).astype(np.float32).astype(np.float64) * inv_t).astype(np.float32)
    r = rng.uniform(float(pt.astype(np.float64).sum()))
    for w, i in zip(pt, order[:keep]):
        r -= float(w)
        if r <= 0.0:
            return int(i)
    return int(order[keep - 1])
