"""Sampling: parameters, the reference's generator and chain, device kernels."""
from .params import GenerateParams, GenerateResult, SamplerParams, StopReason
from .rng import Mt19937_64
from .chain import argmax_first, sample_from_candidates, sample_from_logits
from .sampler import Sampler

__all__ = ["GenerateParams", "GenerateResult", "SamplerParams", "StopReason", "Mt19937_64", "argmax_first",
           "sample_from_candidates", "sample_from_logits", "Sampler"]
