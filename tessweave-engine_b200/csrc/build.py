"""Compile the ``.cu`` files of this folder with nvcc for sm_100a and load them.

Each source file becomes one shared library of ``extern "C"`` launchers, loaded
with ctypes (no torch headers are involved, so a file compiles in seconds).  A
library's file name carries a hash of its source, of the headers beside it and of
the flags, so a stale binary is never loaded.  Libraries are kept in ``_build/``
beside the sources when that folder can be written, else in a per-user folder
under the system's temporary directory.  Nothing is compiled until a library is
first asked for; while nvcc runs, a line is printed every few seconds.
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

CSRC = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the CUDA "
                     "kernels of this engine cannot be compiled, and there is no fallback path")


def _build_dir() -> Path:
    override = os.environ.get("TESSWEAVE_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(CSRC / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"tessweave_b200_build_{os.getuid()}")
    for cand in candidates:
        try:
            cand.mkdir(parents=True, exist_ok=True)
            probe = cand / f".w{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return cand
        except OSError:
            continue
    raise BuildError("no writable folder for compiled kernels: tried " + ", ".join(map(str, candidates)))


def _digest(source: Path, defines: dict[str, int | str]) -> str:
    h = hashlib.sha1()
    h.update(source.read_bytes())
    for header in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(header.name.encode())
        h.update(header.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(" ".join(ARCH_FLAGS + BASE_FLAGS).encode())
    return h.hexdigest()[:12]


def library_path(name: str, defines: dict[str, int | str] | None = None) -> Path:
    defines = defines or {}
    source = CSRC / f"{name}.cu"
    if not source.exists():
        raise BuildError(f"no kernel source {source}")
    tag = "".join(f"_{k.lower()}{v}" for k, v in sorted(defines.items()))
    return _build_dir() / f"tw_{name}{tag}.{_digest(source, defines)}.so"


def compile_library(name: str, defines: dict[str, int | str] | None = None, verbose: bool = True) -> Path:
    """Compile ``<name>.cu`` (once) and return the path of the shared library."""
    defines = defines or {}
    out = library_path(name, defines)
    if out.exists():
        return out
    source = CSRC / f"{name}.cu"
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [_nvcc(), *ARCH_FLAGS, *BASE_FLAGS, "-I", str(CSRC)]
    cmd += [f"-D{k}={v}" for k, v in sorted(defines.items())]
    cmd += ["-o", str(tmp), str(source)]
    label = out.name
    if verbose:
        print(f"[tessweave] compiling {source.name} for sm_100a -> {label}", file=sys.stderr, flush=True)
    started = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            print(f"[tessweave] still compiling {source.name} ({time.time() - started:.0f} s)",
                  file=sys.stderr, flush=True)

    t = threading.Thread(target=ticker, daemon=True)
    if verbose:
        t.start()
    output, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise BuildError(f"nvcc failed on {source.name}:\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, out)  # atomic: a concurrent process sees either nothing or the whole file
    if verbose:
        print(f"[tessweave] built {label} in {time.time() - started:.1f} s", file=sys.stderr, flush=True)
    return out


def timeline_enabled() -> bool:
    """``TESSWEAVE_TIMELINE=1``: every library is compiled with the device-side timeline (see common.cuh)."""
    return os.environ.get("TESSWEAVE_TIMELINE") == "1"


_timeline_buffer: list[int] = [0]     # device address handed to every library loaded with the timeline


def set_timeline_buffer(address: int) -> None:
    """Hand the timeline buffer (device address; 0 = none) to the loaded libraries and to those loaded later."""
    with _lock:
        _timeline_buffer[0] = address
        for lib in _loaded.values():
            if hasattr(lib, "tw_timeline_set"):
                code = lib.tw_timeline_set(ctypes.c_void_p(address))
                if code != 0:
                    raise BuildError(f"tw_timeline_set failed with CUDA error {code}")


def load_library(name: str, defines: dict[str, int | str] | None = None) -> ctypes.CDLL:
    """The loaded library of ``<name>.cu``; compiled at the first call if need be."""
    if timeline_enabled():
        defines = dict(defines or {}, TW_TIMELINE=1)
    key = name + repr(sorted((defines or {}).items()))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(str(compile_library(name, defines)))
            _loaded[key] = lib
            if _timeline_buffer[0] and hasattr(lib, "tw_timeline_set"):
                lib.tw_timeline_set(ctypes.c_void_p(_timeline_buffer[0]))
        return lib


def all_sources() -> list[str]:
    return sorted(p.stem for p in CSRC.glob("*.cu"))
