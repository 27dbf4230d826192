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
