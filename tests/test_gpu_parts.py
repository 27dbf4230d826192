"""Each part of a layer alone against the plain function of the same part:
norm, position encoding, attention mixer (with and without biases, norms,
window, and on another entry's cache), gated feed-forward, and the pre-norm
block that arranges them.  Sizes differ from the tiny models'."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from gpu_util import DEV, check
from nncpu_b200.cache import Cache
from nncpu_b200.config import AttentionSpec, BlockSpec, GatedMlpSpec, NormSpec, PositionSpec
from nncpu_b200.engine import make_context
from nncpu_b200.parts import EntryCache, Runtime, build
from nncpu_b200.weights import random_tensors

pytestmark = pytest.mark.gpu
RUNS = [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)]


def bound(family, spec, dtype, seed=0, **kw):
    part = build(family, spec, **kw)
    tensors = random_tensors(part.params(), seed, torch.float32, include_optional=True)
    ref = {k: v.to(dtype).float().numpy() for k, v in tensors.items()}
    part.bind({k: v.to(dtype).to(DEV) for k, v in tensors.items()}, Runtime(DEV, dtype))
    return part, ref


def step_context(cache, lens, new):
    """Slots that already hold lens[b] tokens receive new[b] more."""
    slots = [cache.alloc_slot() for _ in lens]
    for s, n in zip(slots, lens):
        if n:
            cache.prepare([s], [n])
            cache.commit([s], [n])
    cache.prepare(slots, new)
    return slots, make_context(cache, slots, [[0] * n for n in new], [[] for _ in new])


@pytest.mark.parametrize("dtype,tol", RUNS)
def test_norm_part(dtype, tol):
    norm, w = bound("norm", NormSpec("rmsnorm", 72, 3e-5, "n"), dtype)
    x = torch.randn(6, 72, device=DEV) * 2
    want = P.rmsnorm(x.cpu().numpy(), w["n.weight"], 3e-5)
    check(norm.forward(None, x), want, tol, "norm")
    rows = torch.tensor([5, 0], dtype=torch.int32, device=DEV)
    check(norm.forward(None, x, rows=rows), want[[5, 0]], tol, "norm of chosen rows")


def test_rope_part_is_shared_within_a_step():
    pos_a, pos_b = (build("position", PositionSpec("rope_neox", 1e4, 32)) for _ in range(2))
    other = build("position", PositionSpec("rope_neox", 1e6, 32))
    rt = Runtime(DEV, torch.float32)
    for p in (pos_a, pos_b, other):
        p.bind({}, rt)
    cache = Cache([], [], 256, torch.float32, DEV)
    _, ctx = step_context(cache, [0, 70], [5, 2])
    t = pos_a.tables(ctx)
    assert pos_b.tables(ctx) is t and other.tables(ctx) is not t      # same encoding: computed once per step
    ang = np.array([0, 1, 2, 3, 4, 70, 71], dtype=np.float32)[:, None] * \
        (1e4 ** (-2.0 * np.arange(16) / 32)).astype(np.float32)[None, :]
    assert np.abs(t[..., 0].cpu().numpy() - np.cos(ang.astype(np.float64))).max() < 2e-6
    assert np.abs(t[..., 1].cpu().numpy() - np.sin(ang.astype(np.float64))).max() < 2e-6


def plain_attention_part(spec, w, x, window, shared_kv=None):
    """One whole sequence through the mixer, written with the plain functions."""
    T, n = x.shape[0], spec.name
    bias = (lambda p: w.get(f"{n}.{p}.bias"))
    q = P.linear(x, w[f"{n}.q_proj.weight"], bias("q_proj")).reshape(T, spec.n_heads, spec.head_dim)
    if shared_kv is None:
        k = P.linear(x, w[f"{n}.k_proj.weight"], bias("k_proj")).reshape(T, spec.n_kv_heads, spec.head_dim)
        v = P.linear(x, w[f"{n}.v_proj.weight"], bias("v_proj")).reshape(T, spec.n_kv_heads, spec.head_dim)
    if spec.qk_norm is not None:
        q = P.rmsnorm(q, w[f"{spec.qk_norm.name}.q_norm.weight"], spec.qk_norm.eps)
        if shared_kv is None:
            k = P.rmsnorm(k, w[f"{spec.qk_norm.name}.k_norm.weight"], spec.qk_norm.eps)
    if spec.position is not None:
        q = P.rope_neox(q, np.arange(T), spec.position.theta, spec.position.rotary_dim)
        if shared_kv is None:
            k = P.rope_neox(k, np.arange(T), spec.position.theta, spec.position.rotary_dim)
    if shared_kv is not None:
        k, v = shared_kv
    a = P.attention(q * (spec.scale * math.sqrt(spec.head_dim)), k, v, window)
    return P.linear(a, w[f"{n}.o_proj.weight"], w.get(f"{n}.o_proj.bias")), (k, v)


VARIANTS = {
    "qwen3-like": dict(n_heads=6, n_kv_heads=2, head_dim=32, qkv_bias=False, window=0, norm=True, rope=True),
    "biases, one kv head": dict(n_heads=3, n_kv_heads=1, head_dim=48, qkv_bias=True, window=0, norm=True, rope=True),
    "window": dict(n_heads=4, n_kv_heads=4, head_dim=16, qkv_bias=False, window=9, norm=True, rope=True),
    "no norm, no position, partial scale": dict(n_heads=2, n_kv_heads=1, head_dim=64, qkv_bias=True, window=0,
                                                norm=False, rope=False, scale=0.2),
    "partial rotation": dict(n_heads=2, n_kv_heads=2, head_dim=32, qkv_bias=False, window=0, norm=True, rope=True,
                             rotary_dim=16),
}


def attention_spec(v, hidden=88):
    return AttentionSpec(kind="attention", name="att", hidden_size=hidden, n_heads=v["n_heads"],
                         n_kv_heads=v["n_kv_heads"], head_dim=v["head_dim"], qkv_bias=v["qkv_bias"],
                         out_bias_optional=v["qkv_bias"], scale=v.get("scale", v["head_dim"] ** -0.5),
                         window=v["window"], qk_norm=NormSpec("rmsnorm", v["head_dim"], 1e-5, "att") if v["norm"] else None,
                         position=PositionSpec("rope_neox", 5e4, v.get("rotary_dim", v["head_dim"])) if v["rope"] else None)


@pytest.mark.parametrize("dtype,tol", RUNS)
@pytest.mark.parametrize("variant", list(VARIANTS))
def test_attention_part(variant, dtype, tol):
    spec = attention_spec(VARIANTS[variant])
    mixer, w = bound("mixer", spec, dtype, seed=3)
    T = 100
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, 88, generator=g).to(dtype)
    want, _ = plain_attention_part(spec, w, x.float().numpy(), spec.window)
    cache = Cache([(mixer.kv_request(), None)], [None], 512, dtype, DEV)
    # prompt of 70 in one step, then 30 tokens in steps of 10: the same rows must come out
    slot = cache.alloc_slot()
    got = []
    for a, b in [(0, 70)] + [(s, s + 10) for s in range(70, 100, 10)]:
        cache.prepare([slot], [b - a])
        ctx = make_context(cache, [slot], [[0] * (b - a)], [[]])
        residual = torch.zeros(b - a, 88, device=DEV)
        k, v = cache.kv(0)
        mixer.forward(ctx, x[a:b].to(DEV), residual, EntryCache(k, v, ctx.block_tables[0], True, None))
        cache.commit([slot], [b - a])
        got.append(residual)
    check(torch.cat(got), want, tol, variant)


@pytest.mark.parametrize("dtype,tol", RUNS)
def test_attention_part_on_another_entrys_cache(dtype, tol):
    v = VARIANTS["qwen3-like"]
    owner_spec = attention_spec(v)
    owner, w_owner = bound("mixer", owner_spec, dtype, seed=4)
    reader, w_reader = bound("mixer", owner_spec, dtype, seed=5, reads_other_cache=True)
    assert reader.kv_request() is None and "att.k_proj.weight" not in w_reader and "att.k_norm.weight" not in w_reader
    T = 40
    x = torch.randn(T, 88).to(dtype)
    y = torch.randn(T, 88).to(dtype)
    _, kv = plain_attention_part(owner_spec, w_owner, x.float().numpy(), 0)
    kv = tuple(P.f32_to_bf16_f32(t) if dtype == torch.bfloat16 else t for t in kv)
    want, _ = plain_attention_part(owner_spec, w_reader, y.float().numpy(), 0, shared_kv=kv)
    cache = Cache([(owner.kv_request(), None), (None, None)], [None, 0], 128, dtype, DEV)
    slot = cache.alloc_slot()
    cache.prepare([slot], [T])
    ctx = make_context(cache, [slot], [[0] * T], [[]])
    k, vv = cache.kv(0)
    owner.forward(ctx, x.to(DEV), torch.zeros(T, 88, device=DEV), EntryCache(k, vv, ctx.block_tables[0], True, None))
    residual = torch.zeros(T, 88, device=DEV)
    k2, v2 = cache.kv(1)
    before = k2.clone()
    reader.forward(ctx, y.to(DEV), residual, EntryCache(k2, v2, ctx.block_tables[0], False, None))
    assert torch.equal(k2, before)            # a reader appends nothing
    check(residual, want, tol, "reader of another entry's cache")


@pytest.mark.parametrize("dtype,tol", RUNS)
def test_feed_forward_part(dtype, tol):
    spec = GatedMlpSpec(kind="gated_mlp", name="ff", hidden_size=72, intermediate_size=200, activation="silu")
    ff, w = bound("feed_forward", spec, dtype, seed=6)
    x = torch.randn(9, 72).to(dtype)
    xf = x.float().numpy()
    want = P.linear(P.swiglu(P.linear(xf, w["ff.gate_proj.weight"]), P.linear(xf, w["ff.up_proj.weight"])),
                    w["ff.down_proj.weight"])
    residual = torch.ones(9, 72, device=DEV)
    ff.forward(None, x.to(DEV), residual)
    check(residual - 1, want, tol, "feed-forward adds to the residual")


@pytest.mark.parametrize("dtype,tol", RUNS)
def test_prenorm_block(dtype, tol):
    a = attention_spec(VARIANTS["biases, one kv head"])
    spec = BlockSpec("prenorm", NormSpec("rmsnorm", 88, 1e-6, "n1"), a, NormSpec("rmsnorm", 88, 2e-6, "n2"),
                     GatedMlpSpec(kind="gated_mlp", name="ff", hidden_size=88, intermediate_size=120))
    block, w = bound("block", spec, dtype, seed=7)
    T = 30
    x0 = torch.randn(T, 88)
    r = lambda t: P.f32_to_bf16_f32(t) if dtype == torch.bfloat16 else t
    x = x0.numpy()
    att, _ = plain_attention_part(a, w, r(P.rmsnorm(x, w["n1.weight"], 1e-6)), 0)
    x = x + att
    h = r(P.rmsnorm(x, w["n2.weight"], 2e-6))
    x = x + P.linear(P.swiglu(P.linear(h, w["ff.gate_proj.weight"]), P.linear(h, w["ff.up_proj.weight"])),
                     w["ff.down_proj.weight"])
    cache = Cache(block.cache_requests(), [None], 64, dtype, DEV)
    slot = cache.alloc_slot()
    cache.prepare([slot], [T])
    ctx = make_context(cache, [slot], [[0] * T], [[]])
    residual = x0.to(DEV).clone()
    k, v = cache.kv(0)
    block.forward(ctx, residual, [EntryCache(k, v, ctx.block_tables[0], True, None)])
    assert residual.dtype == torch.float32          # the residual stream stays in 32-bit
    check(residual, x, tol, "pre-norm block")
