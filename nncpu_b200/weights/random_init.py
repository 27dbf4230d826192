"""Random-weights mode: a model folder from a configuration and a seed.

Every tensor is drawn from a generator keyed by (seed, tensor name), so a
tensor's values do not depend on which other tensors exist or on the order in
which they are made.  Matrices, tables and biases are N(0, 0.02) and norm
weights 1 + N(0, 0.1); the reference's test models are made the same way with
other widths (crates/nncpu/src/model/tests.rs:18-47,179-194).
"""
from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Dict, Iterable

import numpy as np
import torch

from ..errors import InvalidArgument
from .params import ParamSpec
from .safetensors_io import write_safetensors


def draw(p: ParamSpec, seed: int) -> torch.Tensor:
    """The float32 values of one tensor."""
    key = [int(seed) & 0xFFFFFFFFFFFFFFFF, zlib.crc32(p.name.encode())]
    rng = np.random.Generator(np.random.Philox(key=key))
    kind, std = p.init
    x = rng.standard_normal(size=p.shape, dtype=np.float32) * np.float32(std)
    if kind == "one_plus_normal":
        x += np.float32(1.0)
    elif kind != "normal":
        raise InvalidArgument(f"{p.name}: unknown initialisation {kind!r}")
    return torch.from_numpy(x)


def random_tensors(params: Iterable[ParamSpec], seed: int, store_dtype: torch.dtype = torch.bfloat16,
                   vector_dtype: torch.dtype = None, include_optional: bool = False) -> Dict[str, torch.Tensor]:
    """``store_dtype`` for tensors of two or more axes, ``vector_dtype``
    (default the same) for one-axis tensors such as norm weights and biases."""
    vector_dtype = vector_dtype or store_dtype
    out = {}
    for p in params:
        if not p.required and not include_optional:
            continue
        out[p.name] = draw(p, seed).to(vector_dtype if len(p.shape) < 2 else store_dtype)
    return out


def random_tensors_on_device(params: Iterable[ParamSpec], seed: int, dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    """The same distributions drawn on the GPU, for models too large to be
    worth a round trip through a file (benchmarks at 8B sizes and above).  The
    generator is the device's, keyed by (seed, tensor name); the values are
    not those of ``draw``.  Two-axis tensors are made in ``dtype``, one-axis
    tensors in float32 when ``dtype`` is float32 and in ``dtype`` otherwise."""
    out = {}
    gen = torch.Generator(device=device)
    for p in params:
        if not p.required:
            continue
        gen.manual_seed((int(seed) * 1000003 + zlib.crc32(p.name.encode())) & 0x7FFFFFFFFFFFFFFF)
        kind, std = p.init
        t = torch.empty(p.shape, dtype=dtype, device=device)
        t.normal_(0.0, std, generator=gen)
        if kind == "one_plus_normal":
            t += 1.0
        out[p.name] = t
    return out


def write_model_folder(folder, config, seed: int, store_dtype: torch.dtype = torch.bfloat16,
                       vector_dtype: torch.dtype = None, include_optional: bool = False) -> Path:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` (a
    registered architecture's configuration object) and returns the folder."""
    from ..engine.model import parameter_list
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}.get(store_dtype, str(store_dtype))
    (folder / "config.json").write_text(json.dumps(d, indent=2) + "\n")
    tensors = random_tensors(parameter_list(config.model_spec()), seed, store_dtype, vector_dtype,
                             include_optional)
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return folder
