"""Weights by tensor name, with one error that says everything that is wrong.

The model lists the tensors its parts need (``ParamSpec``); the loader
compares that list with the file before it reads a byte of data and raises a
single ``BadFormat`` naming every missing tensor, every tensor nobody asked
for and every wrong shape.  The reference refuses the same three ways, one at
a time: a missing tensor (crates/nncpu/src/model/load.rs:406-411), a wrong
shape (crates/nncpu/src/model/load.rs:382-404) and a left-over tensor in a
Qwen file (crates/nncpu/src/model/load.rs:1224-1242).

Element types: with ``dtype=torch.bfloat16`` a tensor stored as BF16 stays
BF16, one stored in 32-bit floats stays in 32-bit floats, F16 becomes BF16,
and integer tables become int32.  With ``dtype=torch.float32`` every floating
tensor is widened to float32 (exact for BF16 and F16).
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Iterable, Optional

import torch

from ..errors import BadFormat
from .params import ParamSpec
from .safetensors_io import SafetensorsFile

_FLOATS = ("F32", "BF16", "F16", "F64")


def check_tensors(file_shapes: Dict[str, tuple], params: Iterable[ParamSpec], where: str) -> None:
    """Raises one BadFormat listing missing, unexpected and mis-shaped tensors."""
    wanted = {p.name: p for p in params}
    missing = sorted(n for n, p in wanted.items() if p.required and n not in file_shapes)
    unexpected = sorted(n for n in file_shapes if n not in wanted)
    wrong = sorted((n, tuple(file_shapes[n]), tuple(p.shape)) for n, p in wanted.items()
                   if n in file_shapes and tuple(file_shapes[n]) != tuple(p.shape))
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where} does not hold the tensors this model needs:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " + ", ".join(
            f"{n} is {list(have)}, expected {list(want)}" for n, have, want in wrong))
    raise BadFormat("\n".join(lines))


def convert(t: torch.Tensor, st_dtype: str, dtype: torch.dtype) -> torch.Tensor:
    """The element-type rule of this module's header, on a CPU tensor."""
    if st_dtype in _FLOATS:
        if dtype == torch.float32 or st_dtype in ("F32", "F64"):
            return t.to(torch.float32)
        return t.to(torch.bfloat16)
    return t.to(torch.int32)


def load_tensors(folder, params: Iterable[ParamSpec], dtype: torch.dtype, device,
                 progress=None) -> Dict[str, torch.Tensor]:
    """Checks ``folder/model.safetensors`` against ``params`` and returns the
    tensors on ``device``.  ``progress(done, total)`` may return False to stop."""
    params = list(params)
    path = Path(folder) / "model.safetensors"
    f = SafetensorsFile(path)
    try:
        check_tensors({n: f.shape(n) for n in f.names()}, params, str(path))
        out: Dict[str, torch.Tensor] = {}
        present = [p for p in params if p.name in f.entries]
        for i, p in enumerate(present):
            t = convert(f.tensor(p.name), f.dtype(p.name), dtype)
            out[p.name] = t.to(device, copy=True) if torch.device(device).type == "cpu" else t.to(device)
            if progress is not None and progress(i + 1, len(present)) is False:
                from ..errors import Cancelled
                raise Cancelled("loading was cancelled")
        return out
    finally:
        f.close()
