"""Reading and writing the safetensors container: an 8-byte little-endian
header length, a JSON header {name: {dtype, shape, data_offsets}}, then the
raw little-endian tensor bytes.  Tensors are found by name; the file is
memory-mapped and nothing is copied until a tensor is asked for.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Tuple

import numpy as np
import torch

from ..errors import BadFormat, UnsupportedModel

# safetensors dtype -> (bytes per element, torch dtype of the mapped view)
_DTYPES = {
    "F32": (4, torch.float32),
    "BF16": (2, torch.bfloat16),
    "F16": (2, torch.float16),
    "I32": (4, torch.int32),
    "I64": (8, torch.int64),
    "U8": (1, torch.uint8),
    "I8": (1, torch.int8),
    "I16": (2, torch.int16),
    "F64": (8, torch.float64),
    "BOOL": (1, torch.bool),
}
_TORCH_TO_ST = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16",
                torch.int32: "I32", torch.int64: "I64"}


class SafetensorsFile:
    """The header of one file and lazy access to its tensors."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except FileNotFoundError:
            raise BadFormat(f"{self.path} does not exist") from None
        size = self.path.stat().st_size
        head = self._fh.read(8)
        if len(head) < 8:
            raise BadFormat(f"{self.path}: too short for a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if n > size - 8 or n > (100 << 20):
            raise BadFormat(f"{self.path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise BadFormat(f"{self.path}: the header is not JSON: {e}") from None
        if not isinstance(header, dict):
            raise BadFormat(f"{self.path}: the header is not a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._base = 8 + n
        self._map = None
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                dtype, shape = info["dtype"], tuple(int(s) for s in info["shape"])
                a, b = (int(v) for v in info["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise BadFormat(f"{self.path}: malformed entry for tensor {name!r}") from None
            if dtype not in _DTYPES:
                raise UnsupportedModel(f"{self.path}: tensor {name!r} has dtype {dtype}, which is not supported")
            count = 1
            for s in shape:
                count *= s
            if a < 0 or b < a or self._base + b > size or b - a != count * _DTYPES[dtype][0]:
                raise BadFormat(f"{self.path}: tensor {name!r} ({dtype} {list(shape)}) does not match "
                                f"its bytes [{a}, {b}) in a file of {size} bytes")
            self.entries[name] = (dtype, shape, a, b)

    def names(self):
        return self.entries.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> str:
        return self.entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapped bytes (read-only: copy before writing)."""
        dtype, shape, a, b = self.entries[name]
        if b == a:
            return torch.empty(shape, dtype=_DTYPES[dtype][1])
        if self._map is None:
            self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=b - a, offset=self._base + a)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the mapped array is read-only
            t = torch.from_numpy(raw)
        return t.view(_DTYPES[dtype][1]).reshape(shape)

    def close(self) -> None:
        self._map = None  # live tensor views keep the mapping alive
        self._fh.close()


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Writes CPU tensors under their names, in name order, 8-byte aligned."""
    header, offset, blobs = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        if t.dtype not in _TORCH_TO_ST:
            raise UnsupportedModel(f"cannot store tensor {name!r} of dtype {t.dtype}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _TORCH_TO_ST[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
