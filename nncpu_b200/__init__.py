"""nncpu_b200: a small, whole generation library for one B200.

Everything between a request's tokens and its next token for the Qwen3 dense
decoder, after ZacWalk/nncpu's engine: typed configuration and an
architecture registry, weights by safetensors name, layers put together from
parts, a paged cache with a slot per sequence, one step function, a generation
loop, sampling, and hand-written sm_100a kernels underneath.
"""
from .errors import (BadFormat, Cancelled, ContextFull, ExtensionError, InvalidArgument, NncpuError, OutOfMemory,
                     UnsupportedModel)
from .engine import Engine, Model
from .perf import perf_enable, perf_report, perf_reset, perf_span_ms, perf_totals
from .sampling import GenerateParams, GenerateResult, SamplerParams, StopReason
from .session import CancelHandle, Piece, Session, SessionParams

__version__ = "0.1.0"

__all__ = ["BadFormat", "Cancelled", "ContextFull", "ExtensionError", "InvalidArgument", "NncpuError",
           "OutOfMemory", "UnsupportedModel", "Engine", "Model", "GenerateParams", "GenerateResult", "SamplerParams",
           "StopReason", "CancelHandle", "Piece", "Session", "SessionParams", "perf_enable", "perf_report", "perf_reset",
           "perf_span_ms", "perf_totals", "__version__"]
