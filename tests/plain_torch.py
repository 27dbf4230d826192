"""A second plain Qwen3 dense decoder, independent of ``plain_qwen3.py``.

Two plain implementations guard against a slip that one reading of the
reference would carry into every comparison.  This one is written from the
same formulas of ZacWalk/nncpu (cited per function as ``path:line`` inside that
project) but in another way throughout, and shares no code with the first one
or with the package:

* PyTorch on the CPU in float64 from end to end (the first one keeps float32
  data and widens inside sums), so the two differ by float32 rounding only;
* attention as one masked matrix per head over the whole sequence (the first
  walks token by token over each token's span);
* rotation angles from ``theta ** (-2 i / n)`` directly (the first multiplies
  a ratio up, as the reference does);
* a file reader of its own, through ``numpy.memmap``.

It rests on the formulas only, like the first: the reference is a Rust crate
and cannot be built here.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch

DT = torch.float64


def open_tensors(path) -> dict:
    """name -> float64 tensor for every tensor of a safetensors file (8-byte
    little-endian header length, JSON header, raw data)."""
    path = Path(path)
    head_len = int(np.fromfile(path, dtype="<u8", count=1)[0])
    header = json.loads(path.read_bytes()[8:8 + head_len])
    blob = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + head_len)
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = np.asarray(blob[lo:hi])
        if meta["dtype"] == "BF16":
            wide = np.zeros(raw.size // 2, dtype="<u4")
            wide[:] = raw.view("<u2")
            t = torch.from_numpy((wide << 16).view("<f4").copy())
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(raw.view("<f4").copy())
        elif meta["dtype"] == "F16":
            t = torch.from_numpy(raw.view("<f2").astype("<f4"))
        else:
            continue
        out[name] = t.to(DT).reshape(meta["shape"])
    return out


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight (crates/nncpu/src/kernels/scalar.rs:270-292)."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def rotate(x, theta):
    """Half-split rotary embedding of x [T, heads, n] at positions 0..T-1: the
    pair (x[i], x[i + n/2]) turns by position * theta^(-2i/n)
    (crates/nncpu/src/kernels/mod.rs:687-737)."""
    T, _, n = x.shape
    half = n // 2
    freq = torch.tensor(theta, dtype=DT) ** (-2.0 * torch.arange(half, dtype=DT) / n)
    angle = torch.arange(T, dtype=DT)[:, None] * freq[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    lo, hi = x[..., :half], x[..., half:]
    return torch.cat([lo * cos - hi * sin, lo * sin + hi * cos], dim=-1)


def masked_attention(q, k, v, window):
    """softmax(q k^T / sqrt(n) + mask) v per head, query head h on key/value
    head h // group; the mask lets position t see positions max(0, t + 1 -
    window) .. t, or all of 0 .. t without a window
    (crates/nncpu/src/model/forward.rs:114-160, crates/nncpu/src/model/embed.rs:14-23)."""
    T, heads, n = q.shape
    group = heads // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("thd,uhd->htu", q, k) / math.sqrt(n)
    t = torch.arange(T)
    seen = t[None, :] <= t[:, None]
    if window > 0:
        seen &= t[None, :] > t[:, None] - window
    scores = scores.masked_fill(~seen[None], float("-inf"))
    return torch.einsum("htu,uhd->thd", scores.softmax(-1), v).reshape(T, heads * n)


class TorchQwen3:
    def __init__(self, folder):
        folder = Path(folder)
        self.c = json.loads((folder / "config.json").read_text())
        self.w = open_tensors(folder / "model.safetensors")

    def _windows(self):
        c, n = self.c, self.c["num_hidden_layers"]
        if not (c.get("use_sliding_window") and c.get("sliding_window")):
            return [0] * n
        kinds = c.get("layer_types") or ["sliding_attention" if i >= c.get("max_window_layers", n) else "full_attention"
                                         for i in range(n)]
        return [c["sliding_window"] if kind == "sliding_attention" else 0 for kind in kinds]

    def logits(self, tokens) -> np.ndarray:
        """[T, vocab] for one whole sequence: embedding, pre-norm blocks (attention with biases before the
        per-head norms, per-head q/k norm, rotation; SiLU-gated feed-forward), final norm, output matrix or the
        embedding table when tied (crates/nncpu/src/model/forward.rs:238-324,735-803,948-985)."""
        c, w = self.c, self.w
        heads, kv = c["num_attention_heads"], c.get("num_key_value_heads", c["num_attention_heads"])
        n = c.get("head_dim") or c["hidden_size"] // heads
        eps, theta = c.get("rms_norm_eps", 1e-6), c.get("rope_theta", 10000.0)
        T = len(tokens)
        x = w["model.embed_tokens.weight"][torch.tensor(tokens)]
        for i, window in enumerate(self._windows()):
            p = f"model.layers.{i}."

            def proj(name, inp):
                y = inp @ w[f"{p}{name}.weight"].T
                bias = w.get(f"{p}{name}.bias")
                return y if bias is None else y + bias
            h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
            q = rms_norm(proj("self_attn.q_proj", h).view(T, heads, n), w[p + "self_attn.q_norm.weight"], eps)
            k = rms_norm(proj("self_attn.k_proj", h).view(T, kv, n), w[p + "self_attn.k_norm.weight"], eps)
            v = proj("self_attn.v_proj", h).view(T, kv, n)
            x = x + proj("self_attn.o_proj", masked_attention(rotate(q, theta), rotate(k, theta), v, window))
            h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
            gate = proj("mlp.gate_proj", h)
            x = x + proj("mlp.down_proj", gate * torch.sigmoid(gate) * proj("mlp.up_proj", h))
        x = rms_norm(x, w["model.norm.weight"], eps)
        head = w["model.embed_tokens.weight"] if c.get("tie_word_embeddings") else w["lm_head.weight"]
        return (x @ head.T).numpy()
