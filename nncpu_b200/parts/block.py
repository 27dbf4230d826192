"""Arrangements of parts in a layer.  "prenorm":
x += mixer(norm1(x)); x += feed_forward(norm2(x))
(crates/nncpu/src/model/forward.rs:735-803 without the Gemma post-norms).
The residual stream stays in float32 from the embedding to the final norm.
"""
from __future__ import annotations

from . import base
from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec, reads_other_cache: bool = False):
        self.norm1 = base.build("norm", spec.norm1)
        kwargs = {"reads_other_cache": True} if reads_other_cache else {}
        self.mixer = base.build("mixer", spec.mixer, **kwargs)
        self.norm2 = base.build("norm", spec.norm2)
        self.feed_forward = base.build("feed_forward", spec.feed_forward)
        self._parts = (self.norm1, self.mixer, self.norm2, self.feed_forward)

    def params(self):
        return [p for part in self._parts for p in part.params()]

    def bind(self, tensors, rt):
        self.rt = rt
        for part in self._parts:
            part.bind(tensors, rt)

    def weight_bytes(self):
        return sum(part.weight_bytes() for part in self._parts)

    def cache_requests(self):
        return [(self.mixer.kv_request(), self.mixer.state_request())]

    def forward(self, ctx, residual, caches):
        with self.rt.scope():       # the mixer's temporaries are done with when the feed-forward starts
            self.mixer.forward(ctx, self.norm1.forward(ctx, residual), residual, caches[0])
        with self.rt.scope():
            self.feed_forward.forward(ctx, self.norm2.forward(ctx, residual), residual)
