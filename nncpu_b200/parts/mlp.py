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
    accepts_deferred_norm = True    # x goes to Runtime.linear, which finishes a norm's unfinished output

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
        gate, up = tensors.pop(f"{s.name}.gate_proj.weight"), tensors.pop(f"{s.name}.up_proj.weight")
        # On the tensor-core path the activation runs in the product's epilogue, on the 32-bit
        # accumulators; for that, gate and up rows are interleaved in blocks of 8.
        self.fused = (gate.dtype == up.dtype and s.intermediate_size % 8 == 0
                      and rt.tensor_cores_take(rt.dtype, gate, s.hidden_size))
        if self.fused:
            h = s.hidden_size
            self.w_gate_up = torch.stack([gate.view(-1, 8, h), up.view(-1, 8, h)], dim=1).reshape(-1, h).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        del gate, up
        self.w_down = tensors[f"{s.name}.down_proj.weight"]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    def forward(self, ctx, x, residual):
        s, rt = self.spec, self.rt
        n = x.shape[0]
        act = rt.empty(n, s.intermediate_size)
        if self.fused:
            with rt.phase("ffn_gate_up", self.w_gate_up, n):
                rt.linear(x, self.w_gate_up, None, act, epilogue="swiglu")
        else:
            gate_up = rt.empty(n, 2 * s.intermediate_size)
            with rt.phase("ffn_gate_up", self.w_gate_up, n):
                rt.linear(x, self.w_gate_up, None, gate_up)
            with rt.phase("ffn_act"):
                ops.swiglu(gate_up, act)
        with rt.phase("ffn_down", self.w_down, n):
            # the last write into the residual stream: it may leave the next norm its input
            rt.linear(act, self.w_down, None, residual, accumulate=True, then_norm=getattr(ctx, "next_norm", None))
