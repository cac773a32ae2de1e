"""Compiles the package's CUDA sources for sm_100a and loads them with ctypes.

Each `.cu` file becomes one shared library of `extern "C"` launchers. A library is
compiled the first time something asks for it (so a model compiles only what it
needs), with the `-D` macros its caller gives, and is cached under `_build/` beside
the sources, keyed by a hash of the source text, the shared header and the flags.
If that folder cannot be written (a read-only checkout), a per-user folder under the
temporary directory is used. While nvcc runs, a line is printed to stderr every few
seconds. There is no fallback: if nvcc is missing or the compile fails, loading
raises `KernelBuildError` with the compiler's output.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path

SOURCE_DIR = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "--shared", "-Xcompiler", "-fPIC"]

_loaded: dict[str, ctypes.CDLL] = {}

TIMELINE = int(os.environ.get("OMNIA_TIMELINE") or 0)
"""With OMNIA_TIMELINE=1 in the environment every library is the tracing build (see common.cuh):
kernels stamp the GPU's clock around their wait for the kernel before them, and `timeline()` reads
the marks. With 2, the kernels that carry block traces (OMNIA_TRACE_BLOCK) stamp from every block
as well. A tracing build is a library of its own beside the ordinary one."""


class KernelBuildError(RuntimeError):
    """The CUDA extension could not be compiled or loaded."""


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise KernelBuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin)")


def _build_dir() -> Path:
    preferred = SOURCE_DIR / "_build"
    try:
        preferred.mkdir(exist_ok=True)
        probe = preferred / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"mlx_omnia_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _digest(source: Path, defines: dict[str, object], extra: list[str]) -> str:
    h = hashlib.sha256()
    h.update(source.read_bytes())
    for header in sorted(SOURCE_DIR.glob("*.cuh")):
        h.update(header.read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(ARCH_FLAGS + BASE_FLAGS + extra).encode())
    return h.hexdigest()[:16]


def _with_mode(defines: dict[str, object] | None) -> dict[str, object]:
    defines = dict(defines or {})
    if TIMELINE:
        defines["OMNIA_TIMELINE"] = TIMELINE
    return defines


def library_path(name: str, defines: dict[str, object] | None = None, extra: list[str] | None = None) -> Path:
    defines = _with_mode(defines)
    extra = extra or []
    source = SOURCE_DIR / f"{name}.cu"
    tag = "".join(f"_{k}{v}" for k, v in sorted(defines.items()))
    return _build_dir() / f"libomnia_{name}{tag}_{_digest(source, defines, extra)}.so"


def compile_library(name: str, defines: dict[str, object] | None = None, extra: list[str] | None = None,
                    verbose: bool = True) -> Path:
    """Compile `name`.cu if its library is not there yet; return the library's path."""
    defines = _with_mode(defines)
    extra = extra or []
    target = library_path(name, defines, extra)
    if target.exists():
        return target
    source = SOURCE_DIR / f"{name}.cu"
    partial = target.with_suffix(f".tmp{os.getpid()}.so")
    command = [_nvcc(), *ARCH_FLAGS, *BASE_FLAGS, *extra, *[f"-D{k}={v}" for k, v in sorted(defines.items())],
               "-I", str(SOURCE_DIR), "-o", str(partial), str(source)]
    if verbose:
        print(f"[mlx_omnia_b200] compiling {target.name} for sm_100a ...", file=sys.stderr, flush=True)
    started = time.time()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = process.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[mlx_omnia_b200]   still compiling {name} ({time.time() - started:.0f} s)",
                      file=sys.stderr, flush=True)
    if process.returncode != 0:
        partial.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed for {source.name}:\n{' '.join(command)}\n{output}")
    os.replace(partial, target)
    # Libraries of the same name and macros built from older sources are of no use any more.
    stem = target.name.rsplit("_", 1)[0]
    for stale in target.parent.glob(stem + "_*.so"):
        if stale != target and stale.name.rsplit("_", 1)[0] == stem:
            stale.unlink(missing_ok=True)
    if verbose:
        print(f"[mlx_omnia_b200]   built {target.name} in {time.time() - started:.1f} s", file=sys.stderr, flush=True)
    return target


def load_library(name: str, defines: dict[str, object] | None = None, extra: list[str] | None = None) -> ctypes.CDLL:
    """The compiled library of `name`.cu, compiling it first if need be."""
    key = f"{name}|{sorted((defines or {}).items())}|{extra or []}"
    lib = _loaded.get(key)
    if lib is None:
        path = compile_library(name, defines, extra)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as error:
            raise KernelBuildError(f"could not load {path}: {error}") from error
        _loaded[key] = lib
    return lib


def timeline() -> list[tuple[int, str, int, int, int, int]]:
    """The marks that kernels of a tracing build (OMNIA_TIMELINE) have left since the last call, in
    order of time: (nanoseconds on the GPU's clock, library, source line, phase, block, SM). Phase
    0: block 0 of a kernel reached its wait for the kernel before it; 1: that wait was over; 2 and
    up: a block trace (OMNIA_TRACE_BLOCK in the source), from every block. Synchronise the device first."""
    if not TIMELINE:
        raise KernelBuildError("set OMNIA_TIMELINE=1 before the package is imported to get the tracing build")
    capacity = 65536
    buffer = (ctypes.c_ulonglong * (3 * capacity))()
    marks = []
    for key, lib in _loaded.items():
        take = getattr(lib, "omnia_timeline_take", None)
        if take is None:  # a library none of whose kernels waits
            continue
        take.argtypes, take.restype = [ctypes.c_void_p, ctypes.c_int], ctypes.c_int
        count = take(buffer, capacity)
        if count < 0:
            raise KernelBuildError(f"could not read the marks of {key}")
        name = key.split("|")[0]
        for i in range(count):
            tag, where = int(buffer[3 * i + 1]), int(buffer[3 * i + 2])
            marks.append((int(buffer[3 * i]), name, tag // 8, tag % 8, where & 0xFFFFFFFF, where >> 32))
    return sorted(marks)
