"""Compiling the CUDA sources of ``csrc/`` into one shared library for sm_100a.

The library has a plain C interface (``extern "C"`` launchers that take raw pointers and a
stream) and is loaded with ctypes, so it needs no Python or torch headers and compiles in
seconds per file. It is built into ``csrc/_build/`` of this checkout at first use; a
read-only checkout falls back to a folder under the system's temporary directory.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

SOURCE_DIR = Path(__file__).resolve().parent.parent / "csrc"
LIBRARY_NAME = "libmlxone_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--threads", "2"]


class KernelBuildError(RuntimeError):
    """The CUDA extension could not be compiled or loaded."""


def _say(message: str) -> None:
    print(f"[mlx-one_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = [os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for candidate in candidates:
        if candidate and Path(candidate).is_file():
            return candidate
    raise KernelBuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                           "the engine has no fallback without its CUDA kernels")


def sources() -> list[Path]:
    return sorted(SOURCE_DIR.glob("*.cu"))


def _fingerprint() -> str:
    digest = hashlib.sha256()
    for path in sorted(SOURCE_DIR.glob("*.cu")) + sorted(SOURCE_DIR.glob("*.cuh")) + \
            sorted(SOURCE_DIR.glob("*.h")):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return digest.hexdigest()[:16]


def _build_dir() -> Path:
    preferred = SOURCE_DIR / "_build"
    try:
        preferred.mkdir(parents=True, exist_ok=True)
        probe = preferred / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"mlx-one_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def library_path(build: bool = True, verbose: bool = True) -> Path:
    """Path of an up-to-date library, compiling what is stale."""
    folder = _build_dir()
    stamp = folder / "fingerprint.txt"
    library = folder / LIBRARY_NAME
    fingerprint = _fingerprint()
    if library.is_file() and stamp.is_file() and stamp.read_text().strip() == fingerprint:
        return library
    if not build:
        raise KernelBuildError(f"{library} is missing or stale")
    nvcc = find_nvcc()
    files = sources()
    if verbose:
        _say(f"compiling {len(files)} CUDA files for sm_100a into {folder} (first use only)")
    started = time.time()

    def compile_one(path: Path) -> Path:
        obj = folder / (path.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(SOURCE_DIR), "-c", str(path), "-o",
               str(obj)]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {path.name}:\n{result.stdout}{result.stderr}")
        if verbose:
            _say(f"  compiled {path.name} ({time.time() - started:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objects = list(pool.map(compile_one, files))
    temporary = folder / f".{LIBRARY_NAME}.{os.getpid()}"
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(temporary), *map(str, objects)]
    result = subprocess.run(link, capture_output=True, text=True)
    if result.returncode != 0:
        raise KernelBuildError(f"linking {LIBRARY_NAME} failed:\n{result.stdout}{result.stderr}")
    os.replace(temporary, library)
    stamp.write_text(fingerprint)
    if verbose:
        _say(f"built {library.name} in {time.time() - started:.0f} s")
    return library
