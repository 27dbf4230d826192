"""The interfaces of the parts a layer is put together from, and the
registries that map a spec's ``kind`` to its implementation.

A part is built from its spec alone (sizes and constants are the spec's
fields), lists the tensors it needs, receives them, and then runs on whatever
step it is given.  No part knows which model it is in.

Adding a part: subclass the interface, decorate the class with the matching
``register_*("kind")``, and emit a spec with that ``kind`` from a
configuration class.  Nothing else changes.

Interfaces (``ctx`` is the engine's ``StepContext``; ``x`` is ``[n_tokens,
hidden]`` in the run's element type; ``residual`` is the float32 residual
stream ``[n_tokens, hidden]``):

* ``Norm.forward(ctx, residual, rows=None) -> x``; optionally ``Norm.request(ctx, residual)`` (see
  ``NormRequest``: at a few tokens a norm can ride on the products around it instead of being a launch)
* ``Mixer.forward(ctx, x, residual, cache) -> None`` adds its output to
  ``residual``; ``cache`` is the ``EntryCache`` of the schedule entry.  A mixer
  asks for storage with ``kv_request()`` / ``state_request()``.
* ``FeedForward.forward(ctx, x, residual) -> None`` adds its output to ``residual``.
* ``PositionEncoding.tables(ctx)`` gives what its mixers need for the step's
  positions, computed once per step.
* ``Block.cache_requests()`` lists what its mixers keep from step to step, one
  ``(KVRequest or None, StateRequest or None)`` pair per mixer (a block may have
  one, several or none); ``Block.forward(ctx, residual, caches) -> None`` runs its
  parts in its arrangement, ``caches[k]`` being the ``EntryCache`` of request ``k``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch

from ..cache import KVRequest, StateRequest
from ..errors import UnsupportedModel
from ..weights.params import ParamSpec


class Part:
    """Common life cycle: ``params()`` before loading, ``bind()`` after."""

    def params(self) -> List[ParamSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        """Takes the tensors it listed (absent optional ones are missing from
        the dict).  ``rt`` is the ``Runtime``: device, element type, kernels."""

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads, for the bandwidth model."""
        return 0


class Norm(Part):
    def forward(self, ctx, residual: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def request(self, ctx, residual: torch.Tensor) -> Optional["NormRequest"]:
        """A request that whoever writes ``residual`` last before this norm reads it leaves the norm's input as
        a by-product, or None if this norm (or this step) has no such short cut."""
        return None


@dataclass
class NormRequest:
    """Handed down through ``ctx.next_norm`` to the part that writes the residual stream last before ``norm``
    reads it.  A part that can fulfil it passes it to ``Runtime.linear(..., then_norm=request)`` with that last
    write and only with it; ``result`` is then a ``DeferredNorm``.  A part that ignores it loses nothing."""
    norm: "Norm"
    residual: torch.Tensor
    gamma: torch.Tensor
    eps: float
    size: int
    result: Optional["DeferredNorm"] = None


@dataclass
class DeferredNorm:
    """A norm's output that is not finished: ``x_gamma`` [n, size] holds residual * gamma in the run's element
    type and ``bins`` the exact accumulators of the sums of squares of the residual's rows.  ``Runtime.linear`` takes
    it in place of a tensor: the few-token product turns the sums into the rows' scales and applies them in its
    epilogue; any other path first makes the ordinary tensor with ``finish()``.  Only parts that set
    ``accepts_deferred_norm`` are given one."""
    x_gamma: torch.Tensor
    bins: torch.Tensor
    request: NormRequest

    @property
    def shape(self):
        return self.x_gamma.shape

    @property
    def dtype(self):
        return self.x_gamma.dtype

    def finish(self, ctx=None) -> torch.Tensor:
        """The norm's output as an ordinary tensor (the norm's own kernel on the residual it was asked for)."""
        return self.request.norm.forward(ctx, self.request.residual)


class PositionEncoding(Part):
    """``tables(ctx)`` gives float32 [n_tokens, half, 2]: for every token of the
    step the (cos, sin) that rotate the pairs (i, i + half) of a head's first
    2 * half dimensions.  An encoding that sets ``tables_by_pair`` also takes
    ``tables(ctx, by_pair=True)`` and gives the same values as [half, n_tokens, 2],
    which the fused q/k/v epilogue of long prompts reads; without it the
    unfused kernels are used."""
    tables_by_pair = False

    def tables(self, ctx):
        raise NotImplementedError


@dataclass
class EntryCache:
    """What one schedule entry sees of the cache during a step."""
    k_pages: Optional[torch.Tensor]      # [n_pages, n_kv_heads, PAGE, head_dim] or None
    v_pages: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]  # int32 [n_seqs, width]: page ids of the step's sequences
    owns_kv: bool                        # False: the pages belong to another entry; read, do not append
    state: Optional[torch.Tensor]        # [n_slots, *shape] or None; index with ctx.seq_slots


class Mixer(Part):
    accepts_deferred_norm = False      # whether ``x`` may be a DeferredNorm (it is then passed to Runtime.linear)

    def kv_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor, cache: EntryCache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    accepts_deferred_norm = False      # whether ``x`` may be a DeferredNorm (it is then passed to Runtime.linear)

    def forward(self, ctx, x: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Block(Part):
    def entry_norm_request(self, ctx, residual: torch.Tensor) -> Optional[NormRequest]:
        """The request of the norm this block begins with, for the block before it to fulfil (None: none)."""
        return None

    def cache_requests(self) -> List[tuple]:
        """One (KVRequest or None, StateRequest or None) pair per mixer of the block, in the order in which
        ``forward`` finds their caches."""
        return []

    def forward(self, ctx, residual: torch.Tensor, caches: List[EntryCache]) -> None:
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, Callable]] = {"norm": {}, "position": {}, "mixer": {}, "feed_forward": {},
                                               "block": {}}


def _register(family: str, kind: str):
    def deco(cls):
        _REGISTRIES[family][kind] = cls
        return cls
    return deco


def register_norm(kind: str):
    return _register("norm", kind)


def register_position(kind: str):
    return _register("position", kind)


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_feed_forward(kind: str):
    return _register("feed_forward", kind)


def register_block(kind: str):
    return _register("block", kind)


def build(family: str, spec, **kwargs):
    """The part registered for ``spec.kind`` in ``family``, built from ``spec``."""
    try:
        cls = _REGISTRIES[family][spec.kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "none"
        raise UnsupportedModel(f"no {family} of kind {spec.kind!r} is registered (registered: {known})") from None
    return cls(spec, **kwargs)
