"""The plain implementation checked against first principles (no GPU): each part
against a formula written another way, and whole-model properties."""
import math

import numpy as np
import torch

import plain_qwen3 as P
from tiny import make_folder


def test_rmsnorm_formula():
    rs = np.random.RandomState(0)
    x = rs.randn(5, 37).astype(np.float32)
    g = (1 + 0.1 * rs.randn(37)).astype(np.float32)
    want = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-5) * g
    assert np.allclose(P.rmsnorm(x, g, 1e-5), want, rtol=1e-6, atol=1e-7)
    assert np.allclose(P.rmsnorm(np.zeros((1, 8), np.float32), np.ones(8, np.float32), 1e-6), 0.0)


def test_rope_is_a_rotation_by_position_differences():
    rs = np.random.RandomState(1)
    hd = 32
    q, k = rs.randn(1, 1, hd).astype(np.float32), rs.randn(1, 1, hd).astype(np.float32)
    def dot(pq, pk):
        return float((P.rope_neox(q, [pq], 1e4, hd) * P.rope_neox(k, [pk], 1e4, hd)).sum())
    assert abs(dot(5, 3) - dot(105, 103)) < 1e-4           # only the distance matters
    assert np.allclose(P.rope_neox(q, [0], 1e4, hd), q)    # position 0 is the identity
    out = P.rope_neox(q, [7], 1e4, hd)
    assert abs(np.linalg.norm(out) - np.linalg.norm(q)) < 1e-5
    # pair (i, i + half) with angle pos * theta^(-2i/hd), written with complex numbers
    half = hd // 2
    z = (q[0, 0, :half] + 1j * q[0, 0, half:]) * np.exp(1j * 7 * 1e4 ** (-2.0 * np.arange(half) / hd))
    assert np.allclose(out[0, 0, :half], z.real, atol=1e-5) and np.allclose(out[0, 0, half:], z.imag, atol=1e-5)
    # a partial rotation leaves the remaining lanes alone
    part = P.rope_neox(q, [7], 1e4, 16)
    assert np.array_equal(part[..., 16:], q[..., 16:]) and not np.allclose(part[..., :16], q[..., :16])


def test_attention_against_a_masked_softmax():
    rs = np.random.RandomState(2)
    T, nh, nkv, hd = 9, 4, 2, 8
    q, k, v = (rs.randn(T, n, hd).astype(np.float32) for n in (nh, nkv, nkv))
    for window in (0, 3):
        got = P.attention(q, k, v, window).reshape(T, nh, hd)
        for h in range(nh):
            s = q[:, h] @ k[:, h // 2].T / math.sqrt(hd)
            i, j = np.arange(T)[:, None], np.arange(T)[None, :]
            mask = (j <= i) & ((j > i - window) if window else True)
            s = np.where(mask, s, -np.inf)
            w = np.exp(s - s.max(-1, keepdims=True))
            w /= w.sum(-1, keepdims=True)
            assert np.allclose(got[:, h], w @ v[:, h // 2], atol=1e-5)
    assert P.attn_span(0, 7) == (0, 7) and P.attn_span(3, 7) == (5, 7) and P.attn_span(40, 7) == (0, 7)


def test_swiglu_and_linear():
    g = np.array([-3.0, 0.0, 2.0], np.float32)
    u = np.array([2.0, 5.0, -1.0], np.float32)
    want = g / (1 + np.exp(-g)) * u
    assert np.allclose(P.swiglu(g, u), want, atol=1e-6)
    x = np.arange(6, dtype=np.float32).reshape(2, 3)
    w = np.array([[1, 0, 0], [0, 1, 1]], np.float32)
    assert np.array_equal(P.linear(x, w, np.array([10, 20], np.float32)), [[10, 23], [13, 29]])


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.14159], np.float32)
    want = torch.tensor(x).bfloat16().float().numpy()
    assert np.array_equal(P.f32_to_bf16_f32(x), want)


def test_whole_model_is_causal_and_uses_every_option(tmp_path):
    rs = np.random.RandomState(3)
    for name in ("A", "B", "C"):
        m = P.PlainQwen3(make_folder(tmp_path / name, name, seed=4))
        toks = list(rs.randint(0, m.cfg.vocab, size=60))
        full = m.logits(toks)
        assert full.shape == (60, m.cfg.vocab) and np.isfinite(full).all()
        assert np.allclose(m.logits(toks[:31]), full[:31], atol=1e-5)     # later tokens change nothing earlier
        other = list(toks)
        other[0] = (other[0] + 1) % m.cfg.vocab
        changed = np.abs(m.logits(other) - full).max(-1)
        assert changed[0] > 1e-4 and changed[-1] > 1e-7
    assert m.cfg.windows == [40, 0, 40, 0]
    b = P.PlainQwen3(make_folder(tmp_path / "B2", "B", seed=4))
    assert "model.layers.0.self_attn.q_proj.bias" in b.w and "lm_head.weight" in b.w
    # the biases matter
    before = b.logits([1, 2, 3])
    b.w["model.layers.0.self_attn.k_proj.bias"] = b.w["model.layers.0.self_attn.k_proj.bias"] + 1.0
    assert np.abs(b.logits([1, 2, 3]) - before).max() > 1e-5


def test_window_hides_far_keys(tmp_path):
    m = P.PlainQwen3(make_folder(tmp_path / "C", "C", seed=5, layer_types=["sliding_attention"] * 4))
    rs = np.random.RandomState(4)
    a = list(rs.randint(0, m.cfg.vocab, size=200))
    b = list(a)
    b[3] = (b[3] + 7) % m.cfg.vocab
    la, lb = m.logits(a), m.logits(b)
    # four layers of window 40 carry a change at most 4 * 39 = 156 positions forward
    assert np.abs(la[3] - lb[3]).max() > 1e-4
    assert np.abs(la[3 + 156] - lb[3 + 156]).max() > 0.0
    assert np.array_equal(la[3 + 157:], lb[3 + 157:])
    full = P.PlainQwen3(make_folder(tmp_path / "Cf", "C", seed=5, use_sliding_window=False))
    assert np.abs(full.logits(a)[199] - full.logits(b)[199]).max() > 0.0


def test_two_independent_plain_implementations_agree(tmp_path):
    """The oracle against a second plain implementation written another way (float64 PyTorch, masked-matrix
    attention, angles by a direct power, its own file reader) on every tiny configuration: with and without
    biases, tied and untied, windows, one key/value head for five, sizes that are no power of two; float32 and
    bfloat16 files.  They differ by the first one's float32 rounding only."""
    from plain_torch import TorchQwen3
    from tiny import TINY
    rs = np.random.RandomState(8)
    for name in TINY:
        for store in (torch.float32, torch.bfloat16):
            folder = make_folder(tmp_path / f"{name}{store}", name, seed=9, store_dtype=store)
            a, b = P.PlainQwen3(folder), TorchQwen3(folder)
            toks = rs.randint(0, a.cfg.vocab, size=130).tolist()
            la, lb = a.logits(toks), b.logits(toks)
            assert la.shape == lb.shape
            err = np.abs(la - lb).max() / np.abs(lb).max()
            assert err < 5e-6, (name, store, err)
            assert (la.argmax(-1) == lb.argmax(-1)).all()
