"""Compiles the CUDA sources of this folder for sm_100a and loads them.

Each ``<name>.cu`` becomes one shared library with a plain C interface, built with
``nvcc`` at its first use and found again by the hash of its sources and flags.  The
libraries are kept in ``_build/`` beside the sources when that folder can be written,
else in a per-user folder under the system's temporary directory.  A library that is
missing and cannot be built is an error: there is no other implementation to fall
back to.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import Dict, Sequence

SOURCE_DIR = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS: Sequence[str] = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
    "--expt-relaxed-constexpr",
)

#: every library of the package; ``build_all`` compiles each of them
LIBRARIES: Sequence[str] = ("elementwise", "rope_kv", "attention", "gemm_f32", "sampling", "attention_noalloc",
                            "attention_decode", "attention_prefill", "gemm_bf16",
                            "attention_prefill_tc", "host_core", "gemm_bf16_pair", "step_exec", "plain_reference")

_loaded: Dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[sglang_rs_b200] {message}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for candidate in (os.environ.get("SRB_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise KernelBuildError("nvcc was not found (looked at $SRB_NVCC, PATH and /usr/local/cuda/bin); "
                           "the CUDA kernels cannot be built and there is no fallback")


def _headers() -> list[str]:
    return sorted(os.path.join(SOURCE_DIR, n) for n in os.listdir(SOURCE_DIR) if n.endswith((".cuh", ".h")))


def _digest(name: str, defines: Sequence[str] = ()) -> str:
    h = hashlib.sha256()
    for path in [os.path.join(SOURCE_DIR, f"{name}.cu"), *_headers()]:
        with open(path, "rb") as handle:
            h.update(handle.read())
    h.update(" ".join([*NVCC_FLAGS, *(f"-D{d}" for d in defines)]).encode())
    return h.hexdigest()[:16]


def build_dir() -> str:
    override = os.environ.get("SRB_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(SOURCE_DIR, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"sglang_rs_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {candidates}")


def _file_name(name: str, defines: Sequence[str] = ()) -> str:
    # a variant built with preprocessor definitions carries them in its name, apart from the plain build
    stem = name if not defines else name + "+" + "+".join(defines)
    return f"{stem}-{_digest(name, defines)}.so"


def library_path(name: str, defines: Sequence[str] = ()) -> str:
    return os.path.join(build_dir(), _file_name(name, defines))


def _find_built(name: str, defines: Sequence[str] = ()) -> str | None:
    """A library built earlier for exactly these sources, wherever it may be read."""
    file_name = _file_name(name, defines)
    for folder in (os.environ.get("SRB_BUILD_DIR"), os.path.join(SOURCE_DIR, "_build")):
        if folder and os.path.exists(os.path.join(folder, file_name)):
            return os.path.join(folder, file_name)
    return None


def compile_library(name: str, defines: Sequence[str] = ()) -> str:
    """The path of the library built from ``name``.cu, compiled now if no build of these sources exists.
    ``defines``: preprocessor definitions of a variant (``SRB_TIMELINE``: blocks record when they start, stop
    waiting and leave); a variant is a file of its own and is loaded only where its path is given
    (``SRB_LIBRARY_<NAME>``)."""
    source = os.path.join(SOURCE_DIR, f"{name}.cu")
    if not os.path.exists(source):
        raise KernelBuildError(f"no such kernel source: {source}")
    found = _find_built(name, defines)
    if found:
        return found
    target = library_path(name, defines)
    if os.path.exists(target):
        return target
    lock_path = target + ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.exists(target):
                return target
            _say(f"compiling {name}.cu for sm_100a ...")
            started = time.time()
            partial = f"{target}.{os.getpid()}.tmp"
            command = [_nvcc(), *NVCC_FLAGS, *(f"-D{d}" for d in defines), "-I", SOURCE_DIR, "-o", partial, source]
            process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            while True:
                try:
                    output, _ = process.communicate(timeout=20)
                    break
                except subprocess.TimeoutExpired:
                    _say(f"  still compiling {name}.cu ({time.time() - started:.0f} s)")
            if process.returncode != 0:
                if os.path.exists(partial):
                    os.remove(partial)
                raise KernelBuildError(f"nvcc failed for {name}.cu:\n{' '.join(command)}\n{output}")
            os.replace(partial, target)
            stem = os.path.basename(target).rsplit("-", 1)[0]
            for stale in os.listdir(os.path.dirname(target)):        # builds of older sources of this library
                if stale.startswith(f"{stem}-") and stale.endswith(".so") and stale != os.path.basename(target):
                    try:
                        os.remove(os.path.join(os.path.dirname(target), stale))
                    except OSError:
                        pass
            _say(f"compiled {name}.cu in {time.time() - started:.1f} s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    try:
        os.remove(lock_path)
    except OSError:
        pass
    return target


#: whether kernels that support it are launched with programmatic dependent launch
_pdl = os.environ.get("SRB_PDL", "1") not in ("0", "", "off", "false")


def set_pdl(on: bool) -> None:
    """Switches programmatic dependent launch (a kernel's set-up overlaps the tail of the
    kernel before it) for the libraries that are loaded and for those loaded later."""
    global _pdl
    _pdl = bool(on)
    for library in _loaded.values():
        if hasattr(library, "srb_set_pdl"):
            library.srb_set_pdl(int(_pdl))


def load_library(name: str) -> ctypes.CDLL:
    """The library of ``<name>.cu``.  ``SRB_LIBRARY_<NAME>`` may name a build of the same source made another
    way (the host code built with sanitizers, for instance); it is loaded in place of the one built here."""
    library = _loaded.get(name)
    if library is None:
        library = ctypes.CDLL(os.environ.get(f"SRB_LIBRARY_{name.upper()}") or compile_library(name))
        library.srb_last_error.restype = ctypes.c_char_p
        if hasattr(library, "srb_set_pdl"):
            library.srb_set_pdl(int(_pdl))
        _loaded[name] = library
    return library


def build_all() -> list[str]:
    return [compile_library(name) for name in LIBRARIES]
