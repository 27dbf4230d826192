"""RMSNorm with learned weights: y = x / sqrt(mean(x^2) + eps) * gamma
(crates/nncpu/src/kernels/scalar.rs:270-292), computed in 32-bit."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.params import ParamSpec
from .base import Norm, NormRequest, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec):
        self.size, self.eps, self.name = spec.size, spec.eps, spec.name
        self.gamma = None

    def params(self):
        return [ParamSpec(f"{self.name}.weight", (self.size,), init=("one_plus_normal", 0.1))]

    def bind(self, tensors, rt):
        self.rt = rt
        self.gamma = tensors[f"{self.name}.weight"]

    def forward(self, ctx, residual, rows=None):
        n = residual.shape[0] if rows is None else rows.numel()
        out = self.rt.empty(n, self.size)
        with self.rt.phase("norm"):
            ops.rmsnorm(residual, self.gamma, self.eps, out, rows)
        return out

    def request(self, ctx, residual):
        """In a bfloat16 run the products around this norm can carry it: the few-token products at up to 16
        tokens, the tensor-core products of whole prompts (a launch, and at many tokens a pass over the residual
        stream, less)."""
        if (self.rt.dtype != torch.bfloat16 or self.size % 16 or residual.dtype != torch.float32
                or not self.rt.fuses_norms(ctx.n_tokens, self.size)):
            return None
        return NormRequest(self, residual, self.gamma, self.eps, self.size)
