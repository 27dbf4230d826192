"""Qwen3 dense decoder: ``config.json`` keys to a typed configuration, and
from there to the parts of each layer.

The reference reads the same quantities from GGUF metadata
(crates/nncpu/src/model/load.rs:431-595) and treats Qwen3 as "Llama layers
with per-head Q/K norms" (crates/nncpu/src/model/mod.rs:65-66): pre-norm
RMSNorm blocks, grouped-query attention with per-head q/k RMSNorm and
half-split RoPE, a SiLU-gated feed-forward, and an output matrix that falls
back to the embedding table (crates/nncpu/src/model/mod.rs:367-372).  A layer
may slide over the last ``sliding_window`` keys
(crates/nncpu/src/model/load.rs:493,1147-1165; the reference's own tiny Qwen3
test model does, crates/nncpu/src/model/tests.rs:154-199).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from ..errors import BadFormat, UnsupportedModel
from .registry import register_architecture
from .specs import (AttentionSpec, BlockSpec, EmbeddingSpec, GatedMlpSpec, ModelSpec, NormSpec,
                    OutputSpec, PositionSpec, ScheduleEntry)

_FULL, _SLIDING = "full_attention", "sliding_attention"


def _need_int(d: dict, key: str, default=None, minimum: int = 1) -> int:
    v = d.get(key, default)
    if v is None:
        raise BadFormat(f'config.json has no "{key}"')
    if isinstance(v, bool) or not isinstance(v, int):
        raise BadFormat(f'config.json: "{key}" must be an integer, not {v!r}')
    if v < minimum:
        raise BadFormat(f'config.json: "{key}" is {v}, expected at least {minimum}')
    return v


def _need_float(d: dict, key: str, default) -> float:
    v = d.get(key, default)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise BadFormat(f'config.json: "{key}" must be a positive number, not {v!r}')
    return float(v)


@register_architecture("Qwen3ForCausalLM")
@dataclass
class Qwen3Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    layer_types: Optional[List[str]] = None
    eos_token_id: Tuple[int, ...] = field(default_factory=tuple)
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    # -- config.json ------------------------------------------------------

    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        """Reads the architecture's own keys; keys it does not know are
        ignored.  Missing basics are a format error, as in the reference
        (crates/nncpu/src/model/load.rs:439-445)."""
        heads = _need_int(d, "num_attention_heads")
        hidden = _need_int(d, "hidden_size")
        head_dim = d.get("head_dim")
        if head_dim is None:
            # the reference's fallback: hidden / heads (crates/nncpu/src/model/load.rs:472-475)
            if hidden % heads:
                raise BadFormat(f'config.json has no "head_dim" and hidden_size {hidden} '
                                f"is not a multiple of num_attention_heads {heads}")
            head_dim = hidden // heads
            d = dict(d, head_dim=head_dim)
        rope = d.get("rope_parameters") if isinstance(d.get("rope_parameters"), dict) else {}
        scaling = d.get("rope_scaling") or {}
        rope_type = scaling.get("rope_type", scaling.get("type", rope.get("rope_type", "default")))
        if rope_type not in (None, "default"):
            raise UnsupportedModel(f"rope scaling of type {rope_type!r} is not supported")
        eos = d.get("eos_token_id")
        eos = tuple(eos) if isinstance(eos, list) else (() if eos is None else (eos,))
        for e in eos:
            if isinstance(e, bool) or not isinstance(e, int):
                raise BadFormat(f'config.json: "eos_token_id" holds {e!r}')
        types = d.get("layer_types")
        if types is not None and (not isinstance(types, list) or
                                  any(t not in (_FULL, _SLIDING) for t in types)):
            raise UnsupportedModel(f'config.json: "layer_types" must list "{_FULL}" or "{_SLIDING}"')
        window = d.get("sliding_window")
        cfg = cls(
            hidden_size=hidden,
            num_hidden_layers=_need_int(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=_need_int(d, "num_key_value_heads", heads),
            head_dim=_need_int(d, "head_dim"),
            intermediate_size=_need_int(d, "intermediate_size"),
            vocab_size=_need_int(d, "vocab_size"),
            rms_norm_eps=_need_float(d, "rms_norm_eps", 1e-6),
            rope_theta=_need_float(d, "rope_theta", rope.get("rope_theta", 10000.0)),
            max_position_embeddings=_need_int(d, "max_position_embeddings", 4096),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", False)),
            hidden_act=d.get("hidden_act", "silu"),
            use_sliding_window=bool(d.get("use_sliding_window", False)),
            sliding_window=None if window is None else _need_int(d, "sliding_window"),
            max_window_layers=(None if d.get("max_window_layers") is None
                               else _need_int(d, "max_window_layers", minimum=0)),
            layer_types=types,
            eos_token_id=eos,
            bos_token_id=d.get("bos_token_id"),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "hidden_act": self.hidden_act,
            "use_sliding_window": self.use_sliding_window,
            "torch_dtype": self.torch_dtype,
        }
        # keys without a value are left out, so that the folder this library writes is one other tools load
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.max_window_layers is not None:
            d["max_window_layers"] = self.max_window_layers
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        if self.eos_token_id:
            d["eos_token_id"] = (self.eos_token_id[0] if len(self.eos_token_id) == 1
                                 else list(self.eos_token_id))
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    def validate(self) -> None:
        """Refusals in the reference's spirit: heads divisible by KV heads
        (crates/nncpu/src/model/load.rs:742-749), an even head size
        (crates/nncpu/src/model/load.rs:678-684)."""
        if self.num_attention_heads % self.num_key_value_heads:
            raise BadFormat(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                            f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise BadFormat(f"head_dim {self.head_dim} is odd: rotary pairs need an even size")
        if self.hidden_act != "silu":
            raise UnsupportedModel(f"hidden_act {self.hidden_act!r} is not supported (supported: silu)")
        if self.layer_types is not None and len(self.layer_types) != self.num_hidden_layers:
            raise BadFormat(f'"layer_types" has {len(self.layer_types)} entries for '
                            f"{self.num_hidden_layers} layers")
        if self.use_sliding_window and any(self.windows()) and not self.sliding_window:
            raise BadFormat('"use_sliding_window" is set but "sliding_window" is missing')
        for e in self.eos_token_id:
            if not 0 <= e < self.vocab_size:
                raise BadFormat(f"eos_token_id {e} is outside the vocabulary [0, {self.vocab_size})")

    # -- derived ------------------------------------------------------------

    def windows(self) -> List[int]:
        """Per layer: 0 for every earlier key, else the number of keys the
        layer looks back over."""
        n = self.num_hidden_layers
        if not self.use_sliding_window:
            return [0] * n
        types = self.layer_types
        if types is None:
            first = n if self.max_window_layers is None else self.max_window_layers
            types = [_SLIDING if i >= first else _FULL for i in range(n)]
        return [(self.sliding_window or 0) if t == _SLIDING else 0 for t in types]

    def model_spec(self) -> ModelSpec:
        h, eps = self.hidden_size, self.rms_norm_eps
        position = PositionSpec("rope_neox", theta=self.rope_theta, rotary_dim=self.head_dim)
        layers = []
        for i, window in enumerate(self.windows()):
            p = f"model.layers.{i}"
            layers.append(BlockSpec(
                kind="prenorm",
                norm1=NormSpec("rmsnorm", h, eps, f"{p}.input_layernorm"),
                mixer=AttentionSpec(
                    kind="attention", name=f"{p}.self_attn", hidden_size=h,
                    n_heads=self.num_attention_heads, n_kv_heads=self.num_key_value_heads,
                    head_dim=self.head_dim, qkv_bias=self.attention_bias,
                    out_bias_optional=self.attention_bias,
                    scale=1.0 / math.sqrt(self.head_dim), window=window,
                    qk_norm=NormSpec("rmsnorm", self.head_dim, eps, f"{p}.self_attn"),
                    position=position),
                norm2=NormSpec("rmsnorm", h, eps, f"{p}.post_attention_layernorm"),
                feed_forward=GatedMlpSpec(kind="gated_mlp", name=f"{p}.mlp", hidden_size=h,
                                          intermediate_size=self.intermediate_size,
                                          activation=self.hidden_act)))
        return ModelSpec(
            architecture=self.architecture, hidden_size=h, vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=EmbeddingSpec("model.embed_tokens", self.vocab_size, h),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            output=OutputSpec(norm=NormSpec("rmsnorm", h, eps, "model.norm"), name="lm_head",
                              tied=self.tie_word_embeddings, vocab_size=self.vocab_size,
                              hidden_size=h),
            stop_token_ids=tuple(self.eos_token_id))
