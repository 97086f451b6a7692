"""Compiling the CUDA sources of this package for sm_100a and loading them with ctypes.

Each ``.cu`` file becomes one shared library with ``extern "C"`` launchers that take raw
device pointers, sizes and a stream, so the sources need no framework headers and compile in
seconds.  A library is built at its first use (only the files that the running mode needs
are ever built), into ``_build/`` beside the sources when that folder can be written, else
into a per-user temporary folder; the file name carries a hash of the source and the flags,
so an up-to-date library is reused and a stale one is never loaded.  While ``nvcc`` runs, a
line is printed every few seconds.  A missing compiler or a failed build raises; there is
no other code path.
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

SOURCE_DIR = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]

# library name -> source file
LIBRARIES = {
    "elementwise": "elementwise.cu",
    "gemm_simt": "gemm_simt.cu",
    "attention_generic": "attention_generic.cu",
    "gemm_tcgen05": "gemm_tcgen05.cu",
    "attention_bf16": "attention_bf16.cu",
    "attention_tcgen05": "attention_tcgen05.cu",
    "sampling": "sampling.cu",
    "mma_rate": "mma_rate.cu",
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    found = shutil.which("nvcc") or (
        "/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else None
    )
    if found is None:
        raise BuildError("nvcc was not found: the CUDA kernels of mini_engine_b200 cannot be built")
    return found


_build_dir_cached: Path | None = None
_dir_lock = threading.Lock()


def _build_dir() -> Path:
    """``_build`` beside the sources if writable, else a folder under the temp directory."""
    global _build_dir_cached
    with _dir_lock:
        if _build_dir_cached is None:
            _build_dir_cached = _find_build_dir()
        return _build_dir_cached


def _find_build_dir() -> Path:
    override = os.environ.get("MINI_ENGINE_B200_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(SOURCE_DIR / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"mini_engine_b200_build_{os.getuid()}")
    for folder in candidates:
        try:
            folder.mkdir(parents=True, exist_ok=True)
            probe = folder / f".write_probe_{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
            return folder
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {[str(c) for c in candidates]}")


def _source_hash(source: Path) -> str:
    digest = hashlib.sha256()
    digest.update(source.read_bytes())
    for header in sorted(list(SOURCE_DIR.glob("*.cuh")) + list(SOURCE_DIR.glob("*.h"))):
        digest.update(header.read_bytes())
    digest.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return digest.hexdigest()[:16]


def library_path(name: str) -> Path:
    source = SOURCE_DIR / LIBRARIES[name]
    return _build_dir() / f"{name}-{_source_hash(source)}.so"


def compile_library(name: str, verbose: bool = True) -> Path:
    """Build one library if it is not there yet; return its path."""
    source = SOURCE_DIR / LIBRARIES[name]
    target = library_path(name)
    if target.exists():
        return target
    scratch = target.with_suffix(f".tmp{os.getpid()}.so")
    command = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, "-o", str(scratch), str(source)]
    if verbose:
        print(f"[mini_engine_b200] compiling {source.name} for sm_100a ...", file=sys.stderr, flush=True)
    started = time.time()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(10.0):
            if verbose:
                elapsed = time.time() - started
                print(f"[mini_engine_b200] still compiling {source.name} ({elapsed:.0f} s)", file=sys.stderr, flush=True)

    ticker = threading.Thread(target=heartbeat, daemon=True)
    ticker.start()
    output, _ = process.communicate()
    done.set()
    if process.returncode != 0:
        scratch.unlink(missing_ok=True)
        raise BuildError(f"nvcc failed for {source.name}:\n{output}")
    os.replace(scratch, target)  # atomic: a concurrent builder never sees half a file
    for stale in target.parent.glob(f"{name}-*.so"):  # builds of older sources: never loaded again
        if stale != target and ".tmp" not in stale.name:
            stale.unlink(missing_ok=True)
    if verbose:
        print(f"[mini_engine_b200] built {target.name} in {time.time() - started:.1f} s", file=sys.stderr, flush=True)
    return target


def load_library(name: str) -> ctypes.CDLL:
    with _lock:
        if name not in _loaded:
            _loaded[name] = ctypes.CDLL(str(compile_library(name)))
        return _loaded[name]


def build_all(names: list[str] | None = None, verbose: bool = True) -> list[Path]:
    """Compile the named libraries (all by default), several at a time."""
    names = list(names or LIBRARIES)
    results: dict[str, Path | Exception] = {}

    def work(name: str) -> None:
        try:
            results[name] = compile_library(name, verbose)
        except Exception as error:  # noqa: BLE001 - reported below with the library's name
            results[name] = error

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for name in names:
        if isinstance(results[name], Exception):
            raise results[name]
    return [results[n] for n in names]
