"""Error kinds of the library.

One exception class per kind, after the reference's ``ErrorKind``
(crates/nncpu/src/error.rs:5-69): a caller can catch ``NncpuError`` or the
kind it cares about, and ``err.kind`` names the kind as a string.
"""
from __future__ import annotations


class NncpuError(Exception):
    """Base of every error this library raises on purpose."""
    kind = "Error"


class InvalidArgument(NncpuError, ValueError):
    """A call was made with a value that cannot be right."""
    kind = "InvalidArgument"


class BadFormat(NncpuError):
    """A file does not hold what its format promises."""
    kind = "BadFormat"


class UnsupportedModel(NncpuError):
    """A well-formed model that this library does not run."""
    kind = "UnsupportedModel"


class ContextFull(NncpuError):
    """The cache has no room for the tokens of a step."""
    kind = "ContextFull"


class OutOfMemory(NncpuError, MemoryError):
    """Device or host memory ran out."""
    kind = "OutOfMemory"


class Cancelled(NncpuError):
    """The caller asked the running call to stop."""
    kind = "Cancelled"


class ExtensionError(NncpuError, RuntimeError):
    """The CUDA extension is missing, did not build, or a kernel refused its
    sizes.  There is no fallback path: the call fails."""
    kind = "Extension"


class translating_oom:
    """``with translating_oom("what was being made"):`` turns the device allocator's out-of-memory error into
    ``OutOfMemory`` with the sizes in the message, as the reference turns a failed allocation into its
    ``OutOfMemory`` kind (crates/nncpu/src/model/kv.rs:182-187, crates/nncpu/src/model/load.rs:329-335)."""

    def __init__(self, what: str):
        self.what = what

    def __enter__(self):
        return self

    def __exit__(self, kind, err, tb):
        if kind is None:
            return False
        import torch
        if issubclass(kind, torch.OutOfMemoryError):
            said = str(err).split(". GPU")[0][:200]       # the allocator's own sentence with the size it tried
            raise OutOfMemory(f"{self.what}: the device has no room ({said})") from None
        return False
