"""Gated feed-forward: down(act(gate(x)) * up(x)) with act = SiLU
(crates/nncpu/src/model/forward.rs:763-782,
crates/nncpu/src/kernels/scalar.rs:146-150).  gate and up are stored as one
matrix so the input is read once; the result is added to the residual stream.
"""
from __future__ import annotations

import torch

from ..errors import UnsupportedModel
from ..kernels import ops
from ..weights.params import ParamSpec
from .base import FeedForward, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMlp(FeedForward):
    def __init__(self, spec):
        if spec.activation != "silu":
            raise UnsupportedModel(f"{spec.name}: activation {spec.activation!r} is not supported (supported: silu)")
        self.spec = spec

    def params(self):
        s = self.spec
        return [ParamSpec(f"{s.name}.gate_proj.weight", (s.intermediate_size, s.hidden_size)),
                ParamSpec(f"{s.name}.up_proj.weight", (s.intermediate_size, s.hidden_size)),
                ParamSpec(f"{s.name}.down_proj.weight", (s.hidden_size, s.intermediate_size))]

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        self.w_gate_up = torch.cat([tensors.pop(f"{s.name}.gate_proj.weight"),
                                    tensors.pop(f"{s.name}.up_proj.weight")], dim=0).contiguous()
        self.w_down = tensors[f"{s.name}.down_proj.weight"]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def forward(self, ctx, x, residual):
        s, rt = self.spec, self.rt
        n = x.shape[0]
        gate_up = rt.empty(n, 2 * s.intermediate_size)
        rt.linear(x, self.w_gate_up, None, gate_up)
        act = rt.empty(n, s.intermediate_size)
        ops.swiglu(gate_up, act)
        rt.linear(act, self.w_down, None, residual, accumulate=True)
