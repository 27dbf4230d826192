"""Helpers of the GPU tests: tolerances, page tables made by hand, a step context for one part."""
from __future__ import annotations

import numpy as np
import torch

from nncpu_b200.cache import PAGE

DEV = "cuda:0"
# Largest difference allowed, as a fraction of the largest reference value.
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


def rel_err(got, want) -> float:
    got = got.detach().float().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float32)
    want = want.detach().float().cpu().numpy() if isinstance(want, torch.Tensor) else np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), "the result holds NaN or infinity"
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def check(got, want, tol: float, what: str = "") -> None:
    e = rel_err(got, want)
    assert e <= tol, f"{what}: relative error {e:.3e} above {tol:.1e}"


def scatter_pages(n_pages: int, n_kv: int, hd: int, seqs, dtype, seed: int = 0):
    """Random keys and values for sequences of the given lengths, laid out in
    shuffled pages.  Returns (k_pages, v_pages, block_table int32 [B, width],
    k list, v list) with k[b], v[b] float32 [len, n_kv, hd] holding the stored values."""
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g).tolist()
    width = max((n + PAGE - 1) // PAGE for n in seqs)
    table = torch.full((len(seqs), width), -1, dtype=torch.int32)
    kp = torch.zeros(n_pages, n_kv, PAGE, hd, dtype=dtype)
    vp = torch.zeros(n_pages, n_kv, PAGE, hd, dtype=dtype)
    ks, vs = [], []
    for b, n in enumerate(seqs):
        k = torch.randn(n, n_kv, hd, generator=g).to(dtype)
        v = torch.randn(n, n_kv, hd, generator=g).to(dtype)
        for p in range((n + PAGE - 1) // PAGE):
            page = order.pop()
            table[b, p] = page
            rows = slice(p * PAGE, min(n, (p + 1) * PAGE))
            kp[page, :, :rows.stop - rows.start] = k[rows].transpose(0, 1)
            vp[page, :, :rows.stop - rows.start] = v[rows].transpose(0, 1)
        ks.append(k.float())
        vs.append(v.float())
    return kp.to(DEV), vp.to(DEV), table.to(DEV), ks, vs
