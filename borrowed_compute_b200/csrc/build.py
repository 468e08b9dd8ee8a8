"""Builds the kernel library from the .cu files beside this module and loads it.

The library is one shared object of ``extern "C"`` launchers, compiled for sm_100a only
with plain nvcc (no torch headers, so a full build takes well under a minute).  It is
built in-tree (``csrc/_build``) when that folder can be written, else under
``$BC_B200_BUILD_DIR`` or the temporary folder.  A stamp of the sources and flags decides
whether an existing build is still good.  There is no fallback: if the library can be
neither found nor built, loading raises.
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
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libbc_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]
# More flags for a build of one's own (say -DBC_TC_TRACE for time stamps inside the product kernels); such a build
# has another stamp than the plain one, so give it a folder of its own with BC_B200_BUILD_DIR.
NVCC_FLAGS += os.environ.get("BC_B200_NVCC_EXTRA", "").split()
ABI_VERSION = 1

_lib: Optional[ctypes.CDLL] = None


class KernelBuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _stamp() -> str:
    h = hashlib.sha256()
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _nvcc() -> Optional[str]:
    for cand in (os.environ.get("BC_B200_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    return None


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def _candidate_dirs() -> List[str]:
    dirs = []
    if os.environ.get("BC_B200_BUILD_DIR"):
        dirs.append(os.environ["BC_B200_BUILD_DIR"])
    dirs.append(os.path.join(HERE, "_build"))
    dirs.append(os.path.join(tempfile.gettempdir(), f"bc_b200_build_{os.getuid()}"))
    return dirs


def _good(build_dir: str, stamp: str) -> bool:
    try:
        with open(os.path.join(build_dir, "stamp.txt")) as f:
            return f.read().strip() == stamp and os.path.isfile(os.path.join(build_dir, LIB_NAME))
    except OSError:
        return False


def _say(msg: str) -> None:
    print(f"[borrowed_compute_b200] {msg}", file=sys.stderr, flush=True)


def build(force: bool = False, verbose: bool = True) -> str:
    """Compiles what is stale and returns the path of the shared library."""
    stamp = _stamp()
    if not force:
        for d in _candidate_dirs():
            if _good(d, stamp):
                return os.path.join(d, LIB_NAME)
    nvcc = _nvcc()
    if nvcc is None:
        raise KernelBuildError("the kernel library is not built and nvcc was not found (set BC_B200_NVCC or CUDA_HOME)")
    build_dir = next((d for d in _candidate_dirs() if _writable_dir(d)), None)
    if build_dir is None:
        raise KernelBuildError(f"no writable folder for the kernel build among {_candidate_dirs()}")
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {build_dir} (first call only)")
    started = time.time()

    def compile_one(name: str) -> str:
        obj = os.path.join(build_dir, name[:-3] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", HERE, "-c", os.path.join(HERE, name), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            _say(f"  compiled {name} ({time.time() - started:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp_lib = os.path.join(build_dir, f".{LIB_NAME}.{os.getpid()}")
    res = subprocess.run([nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp_lib] + objs, capture_output=True, text=True)
    if res.returncode != 0:
        raise KernelBuildError(f"linking the kernel library failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp_lib, os.path.join(build_dir, LIB_NAME))
    with open(os.path.join(build_dir, "stamp.txt"), "w") as f:
        f.write(stamp + "\n")
    if verbose:
        _say(f"kernel library ready ({time.time() - started:.0f} s)")
    return os.path.join(build_dir, LIB_NAME)


def load() -> ctypes.CDLL:
    """The loaded library; builds it first if need be.  Raises if that cannot be done."""
    global _lib
    if _lib is None:
        path = build()
        lib = ctypes.CDLL(path)
        lib.bc_abi_version.restype = ctypes.c_int
        if lib.bc_abi_version() != ABI_VERSION:
            raise KernelBuildError(f"{path} has ABI {lib.bc_abi_version()}, this package wants {ABI_VERSION}")
        lib.bc_last_error.restype = ctypes.c_char_p
        _lib = lib
    return _lib


def library_path() -> Optional[str]:
    stamp = _stamp()
    for d in _candidate_dirs():
        if _good(d, stamp):
            return os.path.join(d, LIB_NAME)
    return None
