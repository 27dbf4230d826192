"""Building and loading the CUDA libraries.

Each ``csrc/<name>.cu`` becomes ``csrc/_build/lib<name>.so``: compiled with
nvcc for sm_100a the first time something needs it (or when its source
changed), then loaded with ctypes.  A model only builds what it uses: the
float32 path needs ``generic`` alone.  There is no fallback: if a library
cannot be built or loaded the call raises ``ExtensionError``.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path
from typing import Dict

from ..errors import ExtensionError

CSRC = Path(__file__).resolve().parent.parent / "csrc"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared"]
LIBRARIES = ("generic", "gemm_sm100", "linear_skinny", "attention_mma", "attention_tc")

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _say(msg: str) -> None:
    print(f"[nncpu_b200] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("NNCPU_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise ExtensionError("nvcc was not found (looked at $NNCPU_NVCC, PATH and /usr/local/cuda/bin): "
                         "the CUDA kernels cannot be built, and there is no other path")


def _build_dir() -> Path:
    """In the source tree when it can be written, else a per-user temporary folder."""
    d = CSRC / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"nncpu_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _fingerprint(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in [CSRC / f"{name}.cu"] + sorted(CSRC.glob("*.cuh")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def library_path(name: str) -> Path:
    return _build_dir() / f"lib{name}.so"


def build(name: str, force: bool = False) -> Path:
    """Compiles ``csrc/<name>.cu`` unless an up-to-date library is there."""
    src = CSRC / f"{name}.cu"
    if not src.exists():
        raise ExtensionError(f"{src} does not exist")
    out = library_path(name)
    stamp = out.with_suffix(".hash")
    want = _fingerprint(name)
    if not force and out.exists() and stamp.exists() and stamp.read_text().strip() == want:
        return out
    tmp = out.with_name(f".{out.name}.{os.getpid()}.tmp")
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(tmp), str(src)]
    _say(f"compiling {src.name} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=str(CSRC))
    while True:
        try:
            log, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {src.name} ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise ExtensionError(f"nvcc failed on {src.name}:\n{log}")
    os.replace(tmp, out)
    stamp.write_text(want + "\n")
    _say(f"built {out.name} in {time.time() - t0:.1f} s")
    return out


def build_all(force: bool = False) -> None:
    for name in LIBRARIES:
        build(name, force)


def load(name: str) -> ctypes.CDLL:
    """The loaded library ``name``, built first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise ExtensionError(f"cannot load {path}: {e}") from None
            err = getattr(lib, f"nncpu_last_error_{name}")
            err.restype = ctypes.c_char_p
            lib.last_error = err
            _loaded[name] = lib
        return lib


def loaded_libraries() -> Dict[str, str]:
    return {k: str(library_path(k)) for k in _loaded}
