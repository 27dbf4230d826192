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

A folder holds either ``model.safetensors`` or, for a checkpoint cut into
several files, ``model.safetensors.index.json`` whose ``weight_map`` names the
file of every tensor; the files are checked as one set of tensors.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterable

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


INDEX_NAME = "model.safetensors.index.json"


def open_checkpoint(folder):
    """The files of the checkpoint in ``folder`` and, for every tensor, the
    file that holds it: ({file name: SafetensorsFile}, {tensor: file name},
    what to call the checkpoint in messages)."""
    folder = Path(folder)
    single, index = folder / "model.safetensors", folder / INDEX_NAME
    if single.exists() or not index.exists():
        f = SafetensorsFile(single)          # a missing file is reported by name
        return {single.name: f}, {n: single.name for n in f.names()}, str(single)
    try:
        weight_map = json.loads(index.read_text())["weight_map"]
        if not isinstance(weight_map, dict) or not all(isinstance(v, str) for v in weight_map.values()):
            raise TypeError
    except (json.JSONDecodeError, UnicodeDecodeError, KeyError, TypeError):
        raise BadFormat(f"{index}: no weight_map of tensor names to file names") from None
    files: Dict[str, SafetensorsFile] = {}
    try:
        for name in sorted(set(weight_map.values())):
            if Path(name).name != name:
                raise BadFormat(f"{index}: file name {name!r} points outside the folder")
            files[name] = SafetensorsFile(folder / name)
        absent = sorted(t for t, name in weight_map.items() if t not in files[name].entries)
        if absent:
            raise BadFormat(f"{index} names tensors that their files do not hold: "
                            + ", ".join(f"{t} ({weight_map[t]})" for t in absent))
        # a tensor that a file holds but the index does not name is still part of the checkpoint
        where = dict(weight_map)
        for name, f in files.items():
            for t in f.names():
                where.setdefault(t, name)
    except Exception:
        for f in files.values():
            f.close()
        raise
    return files, where, f"{index} ({len(files)} files)"


def load_tensors(folder, params: Iterable[ParamSpec], dtype: torch.dtype, device,
                 progress=None) -> Dict[str, torch.Tensor]:
    """Checks the checkpoint in ``folder`` against ``params`` and returns the
    tensors on ``device``.  ``progress(done, total)`` may return False to stop."""
    params = list(params)
    files, where, label = open_checkpoint(folder)
    try:
        check_tensors({n: files[name].shape(n) for n, name in where.items()}, params, label)
        out: Dict[str, torch.Tensor] = {}
        present = [p for p in params if p.name in where]
        for i, p in enumerate(present):
            f = files[where[p.name]]
            t = convert(f.tensor(p.name), f.dtype(p.name), dtype)
            out[p.name] = t.to(device, copy=True) if torch.device(device).type == "cpu" else t.to(device)
            if progress is not None and progress(i + 1, len(present)) is False:
                from ..errors import Cancelled
                raise Cancelled("loading was cancelled")
        return out
    finally:
        for f in files.values():
            f.close()
