"""Builds the CUDA sources of ``csrc/`` for sm_100a into one shared library and loads it.

The library is built in-tree (``csrc/_build/``) the first time it is needed, or in a
per-user folder under the system's temporary directory when the tree is read-only.  A
stamp of the sources and flags decides whether a rebuild is needed.  While it compiles
it prints a progress line every few seconds.  There is no fallback: if ``nvcc`` is
missing or a source fails to compile, loading raises.
"""

from __future__ import annotations

import ctypes
import glob
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import FIRST_COMPLETED, ThreadPoolExecutor, wait

_CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libthing_htn_2026_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

_lock = threading.Lock()
_lib = None


class KernelLibraryError(RuntimeError):
    """The CUDA extension could not be built or loaded; nothing runs without it."""


def _say(message: str) -> None:
    print(f"[thing_htn_2026_b200] {message}", file=sys.stderr, flush=True)


def sources() -> list:
    return sorted(glob.glob(os.path.join(_CSRC, "*.cu")))


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise KernelLibraryError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc); "
                             "the CUDA kernels of this library cannot be built")


def _stamp() -> str:
    digest = hashlib.sha256()
    digest.update(" ".join(NVCC_FLAGS).encode())
    for path in sources() + sorted(glob.glob(os.path.join(_CSRC, "*.cuh"))) + sorted(glob.glob(os.path.join(_CSRC, "*.h"))):
        digest.update(os.path.basename(path).encode())
        with open(path, "rb") as handle:
            digest.update(handle.read())
    return digest.hexdigest()


def _writable_build_dir() -> str:
    in_tree = os.path.join(_CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".probe{os.getpid()}")
        with open(probe, "w") as handle:
            handle.write("ok")
        os.remove(probe)
        return in_tree
    except OSError:
        pass
    fallback = os.path.join(tempfile.gettempdir(), f"thing_htn_2026_b200-build-{os.getuid()}")
    os.makedirs(fallback, exist_ok=True)
    return fallback


def _candidate_dirs() -> list:
    return [os.path.join(_CSRC, "_build"),
            os.path.join(tempfile.gettempdir(), f"thing_htn_2026_b200-build-{os.getuid()}")]


def _up_to_date(build_dir: str, stamp: str) -> bool:
    try:
        with open(os.path.join(build_dir, "stamp")) as handle:
            return handle.read().strip() == stamp and os.path.exists(os.path.join(build_dir, LIB_NAME))
    except OSError:
        return False


def _compile_one(nvcc: str, source: str, obj: str, extra: list) -> None:
    command = [nvcc, *NVCC_FLAGS, *extra, "-I", _CSRC, "-c", source, "-o", obj]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise KernelLibraryError(f"nvcc failed on {os.path.basename(source)}:\n{result.stdout}\n{result.stderr}")
    if extra and result.stderr.strip():
        _say(result.stderr.strip())


def build(force: bool = False, ptxas_verbose: bool = False) -> str:
    """Compile every ``csrc/*.cu`` for sm_100a and link the shared library.  Returns its path."""
    stamp = _stamp()
    if not force and not ptxas_verbose:
        for build_dir in _candidate_dirs():
            if _up_to_date(build_dir, stamp):
                return os.path.join(build_dir, LIB_NAME)
    nvcc = _nvcc()
    build_dir = _writable_build_dir()
    srcs = sources()
    if not srcs:
        raise KernelLibraryError(f"no CUDA sources under {_CSRC}")
    started = time.time()
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {build_dir} (first use only)")
    extra = ["-Xptxas", "-v"] if ptxas_verbose else []
    objects = [os.path.join(build_dir, os.path.basename(s)[:-3] + ".o") for s in srcs]
    done = 0
    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
        futures = {pool.submit(_compile_one, nvcc, s, o, extra): s for s, o in zip(srcs, objects)}
        pending = set(futures)
        while pending:
            finished, pending = wait(pending, timeout=5.0, return_when=FIRST_COMPLETED)
            for f in finished:
                f.result()
                done += 1
            if pending and not finished:
                _say(f"  still compiling: {done}/{len(srcs)} done after {time.time() - started:.0f} s")
    tmp_lib = os.path.join(build_dir, f".{LIB_NAME}.{os.getpid()}")
    link = subprocess.run([nvcc, "-shared", "-o", tmp_lib, *objects, "-gencode", "arch=compute_100a,code=sm_100a"],
                          capture_output=True, text=True)
    if link.returncode != 0:
        raise KernelLibraryError(f"linking {LIB_NAME} failed:\n{link.stdout}\n{link.stderr}")
    os.replace(tmp_lib, os.path.join(build_dir, LIB_NAME))
    with open(os.path.join(build_dir, "stamp"), "w") as handle:
        handle.write(stamp)
    _say(f"built {LIB_NAME} in {time.time() - started:.0f} s")
    return os.path.join(build_dir, LIB_NAME)


def load() -> ctypes.CDLL:
    """The loaded library (built first if needed).  Raises :class:`KernelLibraryError`."""
    global _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                lib = ctypes.CDLL(path)
            except OSError as error:
                raise KernelLibraryError(f"cannot load {path}: {error}") from None
            lib.thn_last_error.restype = ctypes.c_char_p
            if lib.thn_abi_version() != 1:
                raise KernelLibraryError(f"{path}: unexpected ABI version {lib.thn_abi_version()}")
            _lib = lib
        return _lib


def library_path() -> str:
    return build()
