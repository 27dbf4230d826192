"""Generality of the parts: a toy architecture defined here, with a mixer that
keeps fixed-size state of its own per sequence, a feed-forward with routing,
another position encoding, and a schedule that runs a layer twice and lets a
layer read another layer's cache, is registered, built, loaded and stepped
without a change to the library's files, and matches a plain version of itself."""
import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from gpu_util import check
from nncpu_b200 import Engine, Model
from nncpu_b200.cache import StateRequest
from nncpu_b200.config import (AttentionSpec, BlockSpec, EmbeddingSpec, FeedForwardSpec, MixerSpec, ModelSpec,
                               NormSpec, OutputSpec, PositionSpec, ScheduleEntry, register_architecture)
from nncpu_b200.kernels import ops
from nncpu_b200.parts import FeedForward, Mixer, PositionEncoding, register_feed_forward, register_mixer, register_position
from nncpu_b200.weights import ParamSpec, write_safetensors, random_tensors
from nncpu_b200.engine.model import parameter_list

pytestmark = pytest.mark.gpu


# -- toy parts ------------------------------------------------------------------------

@dataclass(frozen=True)
class DecaySpec(MixerSpec):
    hidden_size: int = 0
    decay: float = 0.9


@register_mixer("toy_decay")
class DecayMixer(Mixer):
    """state <- decay * state + x_t; out_t = W state.  The state is a vector per
    sequence in the cache's state area; tokens of a sequence run in order."""

    def __init__(self, spec):
        self.spec = spec

    def params(self):
        return [ParamSpec(f"{self.spec.name}.w.weight", (self.spec.hidden_size, self.spec.hidden_size), init=("normal", 0.1))]

    def bind(self, tensors, rt):
        self.rt, self.w = rt, tensors[f"{self.spec.name}.w.weight"]

    def state_request(self):
        return StateRequest((self.spec.hidden_size,), torch.float32)

    def forward(self, ctx, x, residual, cache):
        # Tensor operations only, on the step's device metadata, so that a captured decode graph replays it:
        # states[t] = decay^(i + 1) * state + sum_{j <= i} decay^(i - j) * x[first + j] for the i-th new token of
        # its sequence.  Padding rows (sequence and slot -1) land on the state area's spare last row.
        n, d = ctx.n_tokens, self.spec.decay
        seq, flat = ctx.tok_seq[:n].long(), torch.arange(n, device=x.device)
        first = ctx.cu_seqlens.long()[seq.clamp(min=0)]                      # first flat token of each token's sequence
        lag = (flat[:, None] - flat[None, :]).clamp(min=0).float()
        same = (seq[:, None] == seq[None, :]) & (flat[None, :] <= flat[:, None])
        mix = torch.where(same, torch.pow(torch.full((), d, device=x.device), lag), torch.zeros((), device=x.device))
        slots = ctx.seq_slots.long()
        start = cache.state[slots][seq]                                      # [n, hidden]; seq -1 -> the last sequence's: unused
        start = torch.where((seq >= 0)[:, None], start, cache.state[-1][None, :])
        carry = torch.pow(torch.full((), d, device=x.device), (flat - first + 1).float())[:, None] * start
        states = mix @ x.float() + carry
        last = ctx.cu_seqlens.long()[1:ctx.n_seqs + 1] - 1
        cache.state[slots] = states[last]
        self.rt.linear(states.to(x.dtype), self.w, None, residual, accumulate=True)


@dataclass(frozen=True)
class RoutedSpec(FeedForwardSpec):
    hidden_size: int = 0
    n_experts: int = 0


@register_feed_forward("toy_routed")
class RoutedFeedForward(FeedForward):
    """Router logits in 32-bit choose one expert matrix per token."""

    def __init__(self, spec):
        self.spec = spec

    def params(self):
        s = self.spec
        return [ParamSpec(f"{s.name}.router.weight", (s.n_experts, s.hidden_size), init=("normal", 1.0))] + \
               [ParamSpec(f"{s.name}.experts.{e}.weight", (s.hidden_size, s.hidden_size), init=("normal", 0.1))
                for e in range(s.n_experts)]

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        self.router = tensors[f"{s.name}.router.weight"].float()
        self.experts = [tensors[f"{s.name}.experts.{e}.weight"] for e in range(s.n_experts)]

    def forward(self, ctx, x, residual):
        logits = torch.empty(x.shape[0], self.spec.n_experts, device=x.device, dtype=torch.float32)
        ops.linear_simt(x, self.router, None, logits)
        choice = logits.argmax(-1)
        for e, w in enumerate(self.experts):             # a toy: every expert sees every token, the choice masks
            out = torch.empty(x.shape[0], self.spec.hidden_size, device=x.device, dtype=torch.float32)
            self.rt.linear(x, w, None, out)
            residual += torch.where((choice == e)[:, None], out, torch.zeros((), device=x.device))


@register_position("toy_alibi_like")
class SlopePositions(PositionEncoding):
    """Not a rotation: scales q by 1 / (1 + position / 100), through the same
    table the attention kernel reads (cos = scale, sin = 0)."""

    def __init__(self, spec):
        self.spec, self.half = spec, spec.rotary_dim // 2

    def bind(self, tensors, rt):
        self.rt = rt

    def tables(self, ctx):
        t = ctx.memo.get("toy_slope")
        if t is None:
            scale = 1.0 / (1.0 + ctx.tok_pos.float() / 100.0)
            t = torch.zeros(ctx.n_tokens, self.half, 2, device=scale.device)
            t[..., 0] = scale[:, None]
            ctx.memo["toy_slope"] = t
        return t


@register_architecture("ToyStatefulForCausalLM")
@dataclass
class ToyConfig:
    hidden: int = 48
    vocab: int = 101
    heads: int = 3
    head_dim: int = 16
    experts: int = 3

    @classmethod
    def from_dict(cls, d):
        return cls(d["hidden"], d["vocab"], d["heads"], d["head_dim"], d["experts"])

    def to_dict(self):
        return {"architectures": ["ToyStatefulForCausalLM"], "hidden": self.hidden, "vocab": self.vocab,
                "heads": self.heads, "head_dim": self.head_dim, "experts": self.experts}

    def model_spec(self):
        h = self.hidden
        norm = lambda n: NormSpec("rmsnorm", h, 1e-5, n)
        att = lambda n: AttentionSpec(kind="attention", name=n, hidden_size=h, n_heads=self.heads, n_kv_heads=1,
                                      head_dim=self.head_dim, scale=self.head_dim ** -0.5,
                                      position=PositionSpec("toy_alibi_like", 0.0, self.head_dim))
        ff = lambda n: RoutedSpec(kind="toy_routed", name=n, hidden_size=h, n_experts=self.experts)
        layers = (
            BlockSpec("prenorm", norm("l0.n1"), DecaySpec(kind="toy_decay", name="l0.mix", hidden_size=h, decay=0.8),
                      norm("l0.n2"), ff("l0.ff")),
            BlockSpec("prenorm", norm("l1.n1"), att("l1.att"), norm("l1.n2"), ff("l1.ff")),
            BlockSpec("prenorm", norm("l2.n1"), att("l2.att"), norm("l2.n2"), ff("l2.ff")),
        )
        # layer 0 runs twice (a state of its own each time); layer 2 reads layer 1's keys and values
        schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2, cache_of=1), ScheduleEntry(0))
        return ModelSpec("ToyStatefulForCausalLM", h, self.vocab, 512, EmbeddingSpec("emb", self.vocab, h), layers,
                         schedule, OutputSpec(norm("out"), "head", False, self.vocab, h))


# -- the plain version of the toy -------------------------------------------------------

def plain_toy(cfg, w, tokens):
    T, h = len(tokens), cfg.hidden
    x = w["emb.weight"][np.asarray(tokens)]

    def routed(name, xn):
        choice = (xn.astype(np.float64) @ w[f"{name}.router.weight"].astype(np.float64).T).argmax(-1)
        return np.stack([P.linear(xn[t:t + 1], w[f"{name}.experts.{choice[t]}.weight"])[0] for t in range(T)])

    def decay_layer(x):
        xn = P.rmsnorm(x, w["l0.n1.weight"], 1e-5)
        s, states = np.zeros(h, np.float32), []
        for t in range(T):
            s = np.float32(0.8) * s + xn[t]
            states.append(s)
        x = x + P.linear(np.stack(states), w["l0.mix.w.weight"])
        return x + routed("l0.ff", P.rmsnorm(x, w["l0.n2.weight"], 1e-5))

    def attention_layer(x, name, kv=None):
        xn = P.rmsnorm(x, w[f"{name}.n1.weight"], 1e-5)
        scale = (1.0 / (1.0 + np.arange(T, dtype=np.float32) / np.float32(100.0)))[:, None, None]
        q = P.linear(xn, w[f"{name}.att.q_proj.weight"]).reshape(T, cfg.heads, cfg.head_dim) * scale
        if kv is None:
            k = P.linear(xn, w[f"{name}.att.k_proj.weight"]).reshape(T, 1, cfg.head_dim) * scale
            v = P.linear(xn, w[f"{name}.att.v_proj.weight"]).reshape(T, 1, cfg.head_dim)
            kv = (k, v)
        x = x + P.linear(P.attention(q, kv[0], kv[1], 0), w[f"{name}.att.o_proj.weight"])
        return x + routed(f"{name}.ff", P.rmsnorm(x, w[f"{name}.n2.weight"], 1e-5)), kv

    x = decay_layer(x)
    x, kv = attention_layer(x, "l1")
    x, _ = attention_layer(x, "l2", kv)
    x = decay_layer(x)
    return P.linear(P.rmsnorm(x, w["out.weight"], 1e-5), w["head.weight"])


def test_toy_architecture_is_registered_built_and_stepped(tmp_path):
    cfg = ToyConfig()
    params = parameter_list(cfg.model_spec())
    names = {p.name for p in params}
    assert "l2.att.k_proj.weight" not in names and "l1.att.k_proj.weight" in names      # the reader has no k/v
    tensors = random_tensors(params, 3, torch.float32)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    write_safetensors(tmp_path / "model.safetensors", tensors)
    model = Model.load(tmp_path, dtype="float32")
    engine = Engine(model, max_tokens=512)              # decode steps run as captured graphs
    cache = engine.cache
    assert [s is not None for s in cache.states] == [True, False, False, True]           # a state per run of layer 0
    assert cache.states[0].shape == (cache.n_slots + 1, cfg.hidden)                       # and a spare row for padding
    assert cache.states[0].data_ptr() != cache.states[3].data_ptr()
    assert len(cache.groups) == 1 and cache.groups[0].k.shape[0] == 1 and not cache.owns_kv(2)
    w = {k: v.numpy() for k, v in tensors.items()}
    rs = np.random.RandomState(0)
    a, b, c = rs.randint(0, 101, size=90).tolist(), rs.randint(0, 101, size=37).tolist(), rs.randint(0, 101, size=29).tolist()
    want_a, want_b, want_c = plain_toy(cfg, w, a), plain_toy(cfg, w, b), plain_toy(cfg, w, c)
    sa, sb, sc = engine.alloc_slot(), engine.alloc_slot(), engine.alloc_slot()
    assert sa == 0                                        # a padding row that used slot 0 would spoil a's state
    out = engine.step([sa, sb, sc], [a[:70], b[:5], c[:9]], [list(range(70)), list(range(5)), list(range(9))])
    got_a, got_b, got_c = [out[:70].clone()], [out[70:75].clone()], [out[75:].clone()]
    for i in range(20):                                   # one token each: three live rows in a graph of four,
        out = engine.step([sa, sb, sc], [[a[70 + i]], [b[5 + i]], [c[9 + i]]])   # the state carries on across replays
        got_a.append(out[:1].clone())
        got_b.append(out[1:2].clone())
        got_c.append(out[2:].clone())
    g = engine.graphs.by_size[4]
    assert g.graph is not None and g.n_kernels > 0        # captured at the first of these steps, replayed 19 times
    out = engine.step([sb], [b[25:]], [list(range(12))])  # several tokens at once on a running sequence
    got_b.append(out.clone())
    check(torch.cat(got_a), want_a, 1e-4, "toy model, sequence a")
    check(torch.cat(got_b), want_b, 1e-4, "toy model, sequence b")
    check(torch.cat(got_c), want_c, 1e-4, "toy model, sequence c")
    # a slot that is used again starts from zero state
    engine.free_slot(sa)
    sc = engine.alloc_slot()
    assert sc == sa
    check(engine.step([sc], [b], [list(range(37))]), want_b, 1e-4, "toy model on a reused slot")
