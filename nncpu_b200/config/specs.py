"""Typed descriptions of a model: what each layer is made of, and in which
order layers run.

A configuration class of an architecture turns its ``config.json`` into a
``ModelSpec``.  Everything below the specs (parts, cache, engine) reads sizes
and constants from here and from nowhere else; none of it knows which
architecture it serves.

The reference resolves the same facts per layer at load time into its
``Layer`` records (crates/nncpu/src/model/mod.rs:103-194): head counts, window,
which cache a layer reads, whether it keeps recurrent state.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over a vector of ``size`` lanes, weights at ``name``."""
    kind: str
    size: int
    eps: float
    name: str  # tensor name prefix, e.g. "model.layers.0.input_layernorm"


@dataclass(frozen=True)
class PositionSpec:
    """How positions enter a mixer.  ``kind`` "rope_neox": rotate the pairs
    (i, i + rotary_dim/2) of the first ``rotary_dim`` lanes of a head by
    position * theta^(-2i/rotary_dim)."""
    kind: str
    theta: float
    rotary_dim: int
    position_scale: float = 1.0


@dataclass(frozen=True)
class MixerSpec:
    """The part of a block that looks at other positions.  Subclasses add
    their sizes; ``kind`` picks the implementation from the mixer registry and
    ``name`` is the prefix of its tensors."""
    kind: str
    name: str


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    hidden_size: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    qkv_bias: bool = False
    out_bias_optional: bool = False  # accept "<name>.o_proj.bias" when the file has it
    scale: float = 0.0               # multiplies q.k after the dot product
    window: int = 0                  # 0: every earlier key; n: the last n keys up to the query
    qk_norm: Optional[NormSpec] = None   # per-head norm of q and k (names end in q_norm / k_norm)
    position: Optional[PositionSpec] = None


@dataclass(frozen=True)
class FeedForwardSpec:
    """The part of a block that works on each position alone."""
    kind: str
    name: str


@dataclass(frozen=True)
class GatedMlpSpec(FeedForwardSpec):
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its parts and their arrangement.  ``kind`` "prenorm":
    x += mixer(norm1(x)); x += feed_forward(norm2(x))."""
    kind: str
    norm1: NormSpec
    mixer: MixerSpec
    norm2: NormSpec
    feed_forward: FeedForwardSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers`` and may
    appear in several entries (the layer then runs again with the same
    weights and a cache of its own).  ``cache_of`` names an earlier entry
    whose keys and values this run reads instead of keeping its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    name: str          # tensor name of the table, without ".weight"
    vocab_size: int
    hidden_size: int
    scale: float = 1.0


@dataclass(frozen=True)
class OutputSpec:
    """Final norm and vocabulary projection.  ``tied`` uses the embedding
    table as the output matrix."""
    norm: NormSpec
    name: str          # tensor name of the output matrix, without ".weight"
    tied: bool
    vocab_size: int
    hidden_size: int


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    output: OutputSpec
    stop_token_ids: Tuple[int, ...] = field(default_factory=tuple)
