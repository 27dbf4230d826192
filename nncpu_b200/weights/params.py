"""What a part says about a tensor it needs."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class ParamSpec:
    """``name`` is the full safetensors name.  ``init`` tells the
    random-weights mode how to draw it: ("normal", std) or
    ("one_plus_normal", std)."""
    name: str
    shape: Tuple[int, ...]
    required: bool = True
    init: Tuple[str, float] = ("normal", 0.02)
