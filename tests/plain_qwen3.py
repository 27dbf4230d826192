"""A plain, slow Qwen3 dense decoder on the CPU: whole sequences, no cache.

This file is the oracle of the test suite.  It shares no code with the
package: it parses ``config.json`` and ``model.safetensors`` itself, and every
part of the model is one small numpy function written from the formulas of
ZacWalk/nncpu (cited per function as ``path:line`` inside that project).

It rests on the formulas only: nncpu is a Rust crate and no Rust toolchain is
installed here, so its model code can be neither imported nor compiled and no
golden output of it is committed.

Arithmetic: data are float32; sums of squares, softmax sums and matrix
products are accumulated in float64 and rounded once, which is at least as
exact as the reference (its norms finish in f64, its dot products in f32), so
this side is the more exact one in every comparison.
"""
from __future__ import annotations

import json
import math
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np

F32 = np.float32
F64 = np.float64


# --------------------------------------------------------------------------
# Files
# --------------------------------------------------------------------------

def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns to float32: exact widening
    (crates/nncpu/src/runtime.rs:23-26)."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_f32(x: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16 (ties to even), returned as
    float32 (crates/nncpu/src/runtime.rs:15-21)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def read_safetensors(path) -> dict:
    """Every tensor of a safetensors file as a float32 (or integer) array."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    base = 8 + n
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = raw[base + a:base + b]
        dt = info["dtype"]
        if dt == "F32":
            arr = np.frombuffer(buf, dtype="<f4").astype(F32)
        elif dt == "BF16":
            arr = bf16_bits_to_f32(np.frombuffer(buf, dtype="<u2"))
        elif dt == "F16":
            arr = np.frombuffer(buf, dtype="<f2").astype(F32)
        elif dt == "I32":
            arr = np.frombuffer(buf, dtype="<i4").copy()
        elif dt == "I64":
            arr = np.frombuffer(buf, dtype="<i8").copy()
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = arr.reshape(info["shape"])
    return out


@dataclass
class PlainConfig:
    """The numbers of config.json this oracle needs; the reference reads the
    same ones from GGUF metadata (crates/nncpu/src/model/load.rs:431-595)."""
    n_layer: int
    hidden: int
    n_head: int
    n_kv: int
    head_dim: int
    inter: int
    vocab: int
    eps: float
    theta: float
    tied: bool
    bias: bool
    windows: list  # per layer: 0 = all keys, else the window

    @staticmethod
    def from_file(path) -> "PlainConfig":
        c = json.loads(Path(path).read_text())
        n_layer = c["num_hidden_layers"]
        n_head = c["num_attention_heads"]
        windows = [0] * n_layer
        if c.get("use_sliding_window") and c.get("sliding_window"):
            types = c.get("layer_types")
            if types is None:
                first = c.get("max_window_layers", n_layer)
                types = ["sliding_attention" if i >= first else "full_attention"
                         for i in range(n_layer)]
            windows = [c["sliding_window"] if t == "sliding_attention" else 0 for t in types]
        return PlainConfig(
            n_layer=n_layer, hidden=c["hidden_size"], n_head=n_head,
            n_kv=c.get("num_key_value_heads", n_head),
            head_dim=c.get("head_dim") or c["hidden_size"] // n_head,
            inter=c["intermediate_size"], vocab=c["vocab_size"],
            eps=c.get("rms_norm_eps", 1e-6), theta=c.get("rope_theta", 10000.0),
            tied=bool(c.get("tie_word_embeddings", False)),
            bias=bool(c.get("attention_bias", False)), windows=windows)


# --------------------------------------------------------------------------
# Parts, one function each
# --------------------------------------------------------------------------

def embed(table: np.ndarray, tokens) -> np.ndarray:
    """x[t] = E[token_t] * 1 (crates/nncpu/src/model/forward.rs:897-907; the
    Qwen scale is 1, crates/nncpu/src/model/load.rs:565-566)."""
    return table[np.asarray(tokens, dtype=np.int64)].astype(F32)


def rmsnorm(x: np.ndarray, gamma: np.ndarray, eps: float) -> np.ndarray:
    """y = (x * scale) * gamma over the last axis, with
    scale = f32(1 / sqrt(sum(x^2) * f32(1/dim) + eps)) finished in f64
    (crates/nncpu/src/kernels/scalar.rs:270-292)."""
    dim = x.shape[-1]
    ss = np.sum(x.astype(F64) ** 2, axis=-1, keepdims=True)
    inv_dim = F64(F32(1.0) / F32(dim))
    scale = (1.0 / np.sqrt(ss * inv_dim + F64(F32(eps)))).astype(F32)
    return ((x * scale).astype(F32) * gamma.astype(F32)).astype(F32)


def linear(x: np.ndarray, w: np.ndarray, b=None) -> np.ndarray:
    """y = W x (+ b): rows of W are outputs (crates/nncpu/src/runtime.rs:98-108,
    crates/nncpu/src/model/forward.rs:238-272)."""
    xd = x.astype(F64)
    if w.shape[0] * w.shape[1] > (1 << 26):
        # a large matrix is widened and multiplied a block of outputs at a time (the same sums; less memory)
        y = np.concatenate([xd @ np.asarray(w[i:i + 8192], dtype=F64).T for i in range(0, w.shape[0], 8192)], axis=-1)
    else:
        y = xd @ np.asarray(w, dtype=F64).T
    if b is not None:
        y = y + b.astype(F64)
    return y.astype(F32)


def rope_neox(x: np.ndarray, positions, theta: float, n_rot: int) -> np.ndarray:
    """Half-split rotary embedding of x[t, head, :] at positions[t]:
    ratio = theta^(-2/n_rot), inv_0 = 1, inv_{i+1} = inv_i * ratio in f32,
    angle = f32(pos) * inv_i, pair (x[i], x[i + half])
    (crates/nncpu/src/kernels/mod.rs:687-737)."""
    half = n_rot // 2
    ratio = F32(math.pow(F32(theta), F32(-2.0) / F32(n_rot)))
    inv = np.empty(half, dtype=F32)
    cur = F32(1.0)
    for i in range(half):
        inv[i] = cur
        cur = F32(cur * ratio)
    ang = (np.asarray(positions, dtype=F32)[:, None] * inv[None, :]).astype(F32)
    c = np.cos(ang.astype(F64)).astype(F32)[:, None, :]
    s = np.sin(ang.astype(F64)).astype(F32)[:, None, :]
    out = x.copy()
    a = x[..., :half]
    b = x[..., half:n_rot]
    out[..., :half] = c * a - s * b
    out[..., half:n_rot] = s * a + c * b
    return out.astype(F32)


def attn_span(window: int, pos: int):
    """The keys a causal query at `pos` sees, inclusive: its prefix, or the
    last `window` positions of it (crates/nncpu/src/model/embed.rs:14-23)."""
    first = pos + 1 - window if window > 0 and pos + 1 > window else 0
    return first, pos


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: int) -> np.ndarray:
    """Causal grouped-query attention of one whole sequence.
    q [T, nh, hd], k and v [T, nkv, hd]; query head h reads KV head
    h // (nh / nkv); score = (q . k) * 1/sqrt(hd), scale after the dot;
    softmax over the span; out [T, nh * hd] with heads in order
    (crates/nncpu/src/model/forward.rs:114-160,
    crates/nncpu/src/kernels/scalar.rs:444-548,
    crates/nncpu/src/model/load.rs:538-546)."""
    T, nh, hd = q.shape
    group = nh // k.shape[1]
    scale = F32(1.0 / math.sqrt(hd))
    out = np.zeros((T, nh, hd), dtype=F32)
    for t in range(T):
        first, last = attn_span(window, t)
        for h in range(nh):
            kh = k[first:last + 1, h // group].astype(F64)
            vh = v[first:last + 1, h // group].astype(F64)
            s = (kh @ q[t, h].astype(F64)).astype(F32) * scale
            w = np.exp(s.astype(F64) - F64(s.max()))
            out[t, h] = ((w @ vh) / w.sum()).astype(F32)
    return out.reshape(T, nh * hd)


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """(g * sigmoid(g)) * u with sigmoid(g) = 1 / (1 + exp(-g))
    (crates/nncpu/src/kernels/scalar.rs:102-106,146-150)."""
    g = gate.astype(F64)
    return ((g * (1.0 / (1.0 + np.exp(-g)))).astype(F32) * up).astype(F32)


# --------------------------------------------------------------------------
# Arrangement
# --------------------------------------------------------------------------

class PlainQwen3:
    """Weights by their safetensors names, and the whole forward pass."""

    def __init__(self, folder, round_activations_to_bf16: bool = False):
        folder = Path(folder)
        self.cfg = PlainConfig.from_file(folder / "config.json")
        self.w = read_safetensors(folder / "model.safetensors")
        # With bfloat16 kernels the matrix products read activations rounded
        # to bfloat16; the oracle can round at the same places so that a
        # comparison measures the kernels, not the format.
        self.round = f32_to_bf16_f32 if round_activations_to_bf16 else (lambda a: a)

    def attention_block(self, li: int, x: np.ndarray, positions) -> np.ndarray:
        """Projections, biases before the per-head norms, per-head q/k
        RMSNorm, RoPE on q and k, attention, output projection
        (crates/nncpu/src/model/forward.rs:238-324,434-438)."""
        c, w, p = self.cfg, self.w, f"model.layers.{li}.self_attn."
        T = x.shape[0]
        b = (lambda n: w.get(p + n + ".bias")) if c.bias else (lambda n: None)
        x = self.round(x)
        q = linear(x, w[p + "q_proj.weight"], b("q_proj")).reshape(T, c.n_head, c.head_dim)
        k = linear(x, w[p + "k_proj.weight"], b("k_proj")).reshape(T, c.n_kv, c.head_dim)
        v = linear(x, w[p + "v_proj.weight"], b("v_proj")).reshape(T, c.n_kv, c.head_dim)
        q = rmsnorm(q, w[p + "q_norm.weight"], c.eps)
        k = rmsnorm(k, w[p + "k_norm.weight"], c.eps)
        q = rope_neox(q, positions, c.theta, c.head_dim)
        k = rope_neox(k, positions, c.theta, c.head_dim)
        a = attention(self.round(q), self.round(k), self.round(v), c.windows[li])
        return linear(self.round(a), w[p + "o_proj.weight"], w.get(p + "o_proj.bias"))

    def mlp_block(self, li: int, x: np.ndarray) -> np.ndarray:
        """down(silu(gate(x)) * up(x)) (crates/nncpu/src/model/forward.rs:763-782)."""
        w, p = self.w, f"model.layers.{li}.mlp."
        x = self.round(x)
        act = swiglu(linear(x, w[p + "gate_proj.weight"]), linear(x, w[p + "up_proj.weight"]))
        return linear(self.round(act), w[p + "down_proj.weight"])

    def hidden(self, tokens) -> np.ndarray:
        """Embedding, pre-norm blocks with residual sums, final norm
        (crates/nncpu/src/model/forward.rs:735-762,797-803,948-956)."""
        c, w = self.cfg, self.w
        positions = np.arange(len(tokens))
        x = embed(w["model.embed_tokens.weight"], tokens)
        for li in range(c.n_layer):
            p = f"model.layers.{li}."
            x = x + self.attention_block(li, rmsnorm(x, w[p + "input_layernorm.weight"], c.eps), positions)
            x = x + self.mlp_block(li, rmsnorm(x, w[p + "post_attention_layernorm.weight"], c.eps))
        return rmsnorm(x, w["model.norm.weight"], c.eps)

    def logits(self, tokens, rows=None) -> np.ndarray:
        """Logits [T, vocab] at every position of one whole sequence (or at
        the positions ``rows``); the output matrix is the embedding when the
        file has none (crates/nncpu/src/model/forward.rs:974-985,
        crates/nncpu/src/model/mod.rs:367-372)."""
        w = self.w
        head = w["model.embed_tokens.weight"] if self.cfg.tied else w["lm_head.weight"]
        h = self.hidden(tokens)
        return linear(self.round(h if rows is None else h[list(rows)]), head)


# --------------------------------------------------------------------------
# Choosing a token
# --------------------------------------------------------------------------

def argmax_first(logits: np.ndarray) -> int:
    """The first largest value (crates/nncpu/src/model/forward.rs:1003-1011)."""
    best = 0
    for i in range(1, len(logits)):
        if logits[i] > logits[best]:
            best = i
    return best


class PlainMt19937_64:
    """std::mt19937_64 and the 53-bit uniform the reference draws with
    (crates/nncpu/src/session/sample.rs:8-55)."""
    M64 = (1 << 64) - 1

    def __init__(self, seed: int):
        mt = [seed & self.M64]
        for i in range(1, 312):
            p = mt[-1]
            mt.append((6364136223846793005 * (p ^ (p >> 62)) + i) & self.M64)
        self.mt, self.idx = mt, 312

    def next_u64(self) -> int:
        if self.idx >= 312:
            mt = self.mt
            for i in range(312):
                x = (mt[i] & 0xFFFFFFFF80000000) | (mt[(i + 1) % 312] & 0x7FFFFFFF)
                xa = (x >> 1) ^ (0xB5026F5AA96619E9 if x & 1 else 0)
                mt[i] = mt[(i + 156) % 312] ^ xa
            self.idx = 0
        x = self.mt[self.idx]
        self.idx += 1
        x ^= (x >> 29) & 0x5555555555555555
        x ^= (x << 17) & 0x71D67FFFEDA60000
        x ^= (x << 37) & 0xFFF7EEE000000000
        x ^= x >> 43
        return x & self.M64

    def uniform(self, b: float) -> float:
        return float(self.next_u64() >> 11) * (1.0 / 9007199254740992.0) * b


def sample_chain(logits, rng, temperature: float, top_k: int, top_p: float, min_p: float) -> int:
    """top-k, top-p and min-p on the distribution at temperature 1, then the
    temperature over the survivors and one draw in rank order; NaN counts as
    -inf (crates/nncpu/src/session/sample.rs:69-88,121-201)."""
    cand = [(-math.inf if math.isnan(float(l)) else float(l), i) for i, l in enumerate(logits)]
    cand.sort(key=lambda c: (-c[0], c[1]))
    if 0 < top_k < len(cand):
        cand = cand[:top_k]
    if not cand or not math.isfinite(cand[0][0]):
        return cand[0][1] if cand else 0
    top = cand[0][0]
    prob = [float(F32(math.exp(F32(c[0] - top)))) if c[0] > -math.inf else 0.0 for c in cand]
    total = sum(prob)
    keep = len(cand)
    if 0.0 < top_p < 1.0:
        cum = 0.0
        for i, p in enumerate(prob):
            cum += p / total
            if cum >= float(F32(top_p)):
                keep = i + 1
                break
    if min_p > 0.0:
        floor = float(F32(F32(min_p) * F32(prob[0])))
        i = 1
        while i < keep and prob[i] >= floor:
            i += 1
        keep = i
    inv_t = 1.0 / float(F32(temperature))
    pt = [float(F32(math.exp(float(F32(c[0] - top)) * inv_t))) if c[0] > -math.inf else 0.0
          for c in cand[:keep]]
    r = rng.uniform(sum(pt))
    for p, c in zip(pt, cand):
        r -= p
        if r <= 0.0:
            return c[1]
    return cand[keep - 1][1]
