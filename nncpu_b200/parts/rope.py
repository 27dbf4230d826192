"""Rotary position embedding, half-split pairing (i, i + rotary_dim/2):
angle_i = float32(position) * scale * theta^(-2i/rotary_dim)
(crates/nncpu/src/kernels/mod.rs:687-737).

The inverse frequencies are computed once in float64 and rounded to float32;
the cosines and sines of a step's positions are computed once per step in
32-bit and shared by every layer that uses the same encoding.
"""
from __future__ import annotations

import torch

from ..errors import BadFormat
from ..kernels import ops
from .base import PositionEncoding, register_position


@register_position("rope_neox")
class RopeNeox(PositionEncoding):
    tables_by_pair = True

    def __init__(self, spec):
        if spec.rotary_dim % 2 or spec.rotary_dim <= 0:
            raise BadFormat(f"rotary size {spec.rotary_dim} must be even and positive")
        self.spec = spec
        self.half = spec.rotary_dim // 2
        self.inv_freq = None

    def bind(self, tensors, rt):
        self.rt = rt
        i = torch.arange(self.half, dtype=torch.float64)
        inv = torch.pow(torch.tensor(float(self.spec.theta), dtype=torch.float64), -2.0 * i / self.spec.rotary_dim)
        self.inv_freq = inv.to(torch.float32).to(rt.device)

    def tables(self, ctx, by_pair: bool = False):
        """float32 [n_tokens, half, 2] of (cos, sin), or with ``by_pair`` the same
        values as [half, n_tokens, 2]; memoised in the step."""
        key = ("rope_neox", self.spec, by_pair)
        t = ctx.memo.get(key)
        if t is None:
            shape = (self.half, ctx.n_tokens, 2) if by_pair else (ctx.n_tokens, self.half, 2)
            t = self.rt.empty(*shape, dtype=torch.float32, keep=True)     # every later layer of the step reads it
            ops.rope_table(ctx.tok_pos, self.inv_freq, t, self.spec.position_scale, by_pair)
            ctx.memo[key] = t
        return t
