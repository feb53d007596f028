"""Compile the CUDA sources of ``kvcore_b200/csrc`` into one shared library for sm_100a.

The library is plain C entry points (no Python or torch headers), built with nvcc and
loaded with ctypes, so a fresh checkout compiles in well under a minute.  It is built in
tree (``kvcore_b200/kernels/``) when that folder is writable, else under the system's
temporary folder; the file name carries a hash of the sources and flags, so a stale build
is never loaded.  While nvcc runs, a progress line is printed every few seconds.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_KERNELS_DIR = Path(__file__).resolve().parent
_SRC_DIR = _KERNELS_DIR.parent / "csrc"
_LIB_PREFIX = "libkvcore_b200_sm100a_"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


class KernelBuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    candidates = [
        os.environ.get("KVCORE_NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ]
    for candidate in candidates:
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise KernelBuildError(
        "nvcc was not found (looked at $KVCORE_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin): "
        "the CUDA kernels cannot be compiled, and there is no fallback"
    )


def sources() -> list[Path]:
    return sorted(_SRC_DIR.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(_SRC_DIR.glob("*.cuh")) + list(_SRC_DIR.glob("*.h")))


def source_hash() -> str:
    digest = hashlib.sha256()
    for path in sources() + _headers():
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()[:16]


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".write_probe_{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def _build_dirs() -> list[Path]:
    user = os.getuid() if hasattr(os, "getuid") else 0
    return [_KERNELS_DIR, Path(tempfile.gettempdir()) / f"kvcore_b200_build_{user}"]


def library_path(create_dir: bool = False) -> Path | None:
    """Path of an up-to-date built library, or None if there is none yet."""
    name = _LIB_PREFIX + source_hash() + ".so"
    for folder in _build_dirs():
        candidate = folder / name
        if candidate.is_file():
            return candidate
    return None


def _run(cmd: list[str], label: str, verbose: bool) -> None:
    started = time.time()
    process = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def _progress() -> None:
        while not done.wait(8.0):
            print(f"[kvcore_b200] still compiling {label} ({time.time() - started:.0f}s)",
                  file=sys.stderr, flush=True)

    ticker = threading.Thread(target=_progress, daemon=True)
    ticker.start()
    output, _ = process.communicate()
    done.set()
    if process.returncode != 0:
        raise KernelBuildError(f"nvcc failed on {label}:\n{' '.join(cmd)}\n{output}")
    if verbose and output.strip():
        print(output, file=sys.stderr, flush=True)


def build(verbose: bool = False, extra_flags: list[str] | None = None) -> Path:
    """Compile and link the library if no up-to-date build exists; return its path."""
    existing = library_path()
    if existing is not None:
        return existing
    nvcc = find_nvcc()
    target_dir = next((folder for folder in _build_dirs() if _writable(folder)), None)
    if target_dir is None:
        raise KernelBuildError("no writable folder to build the CUDA kernels in")
    tag = source_hash()
    objects_dir = target_dir / "_build" / tag
    objects_dir.mkdir(parents=True, exist_ok=True)
    lock_path = target_dir / "_build" / "build.lock"
    import fcntl

    with lock_path.open("w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        existing = library_path()
        if existing is not None:  # another process built it while we waited
            return existing
        flags = NVCC_FLAGS + list(extra_flags or [])
        files = sources()
        print(f"[kvcore_b200] compiling {len(files)} CUDA sources for sm_100a into {target_dir}",
              file=sys.stderr, flush=True)
        started = time.time()

        def _compile(src: Path) -> Path:
            obj = objects_dir / (src.stem + ".o")
            _run([nvcc, *flags, "-I", str(_SRC_DIR), "-c", str(src), "-o", str(obj)], src.name, verbose)
            return obj

        with ThreadPoolExecutor(max_workers=min(8, len(files))) as pool:
            objects = list(pool.map(_compile, files))
        library = target_dir / (_LIB_PREFIX + tag + ".so")
        partial = target_dir / (_LIB_PREFIX + tag + f".{os.getpid()}.tmp")
        _run([nvcc, "-Wno-deprecated-gpu-targets", "-shared", "-o", str(partial), *map(str, objects)], "link", verbose)
        os.replace(partial, library)
        for stale in target_dir.glob(_LIB_PREFIX + "*.so"):
            if stale != library:
                try:
                    stale.unlink()
                except OSError:
                    pass
        for stale in (target_dir / "_build").iterdir():  # object files of older source states
            if stale.is_dir() and stale != objects_dir:
                shutil.rmtree(stale, ignore_errors=True)
        print(f"[kvcore_b200] built {library.name} in {time.time() - started:.0f}s",
              file=sys.stderr, flush=True)
        return library


__all__ = ["KernelBuildError", "NVCC_FLAGS", "build", "find_nvcc", "library_path", "source_hash", "sources"]
