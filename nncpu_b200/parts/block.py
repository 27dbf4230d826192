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

    def entry_norm_request(self, ctx, residual):
        return self.norm1.request(ctx, residual) if self.mixer.accepts_deferred_norm else None

    @staticmethod
    def _normed(norm, consumer, ctx, residual, request):
        """``norm``'s output for ``consumer``: what the writer of the residual left, if it fulfilled the request
        of this very norm and the consumer takes it unfinished; else the norm's own kernel."""
        if (request is not None and request.norm is norm and request.result is not None
                and consumer.accepts_deferred_norm):
            return request.result
        return norm.forward(ctx, residual)

    def forward(self, ctx, residual, caches):
        # At a few tokens the norms ride on the products around them: the block before may have left norm1's
        # input (ctx.next_norm), the mixer's last product is asked for norm2's, and the feed-forward's last
        # product for the first norm of the block that follows (ctx.after_block).
        handed, after = ctx.next_norm, ctx.after_block
        ctx.next_norm = ctx.after_block = None
        with self.rt.scope():       # the mixer's temporaries are done with when the feed-forward starts
            x = self._normed(self.norm1, self.mixer, ctx, residual, handed)
            asked = self.norm2.request(ctx, residual) if self.feed_forward.accepts_deferred_norm else None
            ctx.next_norm = asked
            self.mixer.forward(ctx, x, residual, caches[0])
            ctx.next_norm = None
        with self.rt.scope():
            x = self._normed(self.norm2, self.feed_forward, ctx, residual, asked)
            ctx.next_norm = after
            self.feed_forward.forward(ctx, x, residual)
        # ctx.next_norm stays: the block that follows finds its request there, fulfilled or not
