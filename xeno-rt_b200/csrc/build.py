"""Builds the CUDA kernels of this folder into one shared library for sm_100a, in-tree.

Every ``.cu`` file is compiled by ``nvcc -gencode arch=compute_100a,code=sm_100a`` into an object
under ``_build/`` and the objects are linked into ``_build/libxrt_b200_kernels.so``.  A stamp file
holds a hash of the sources and flags; the library is rebuilt when it differs.  The build runs at
the first use of a kernel if the library is missing or stale, prints a line for each file it
compiles, needs no network and no home directory, and uses no Python extension headers, so a
file takes seconds.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

from ..core import KernelError

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libxrt_b200_kernels.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
LINK_LIBS: list[str] = []


def _say(message: str) -> None:
    print(f"[xrt build] {message}", file=sys.stderr, flush=True)


def sources() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cuh") or f.endswith(".h"))


def _source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + LINK_LIBS).encode())
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def find_nvcc() -> str:
    for cand in (os.environ.get("XRT_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelError("nvcc was not found (PATH, /usr/local/cuda/bin, or XRT_NVCC); the CUDA kernels of "
                      "this library cannot be built")


def build_dir() -> str:
    """``_build/`` beside the sources if it can be written, else ``$XRT_BUILD_DIR``, else a folder
    under the system's temporary directory that is named after this checkout."""
    preferred = os.environ.get("XRT_BUILD_DIR") or os.path.join(HERE, "_build")
    try:
        os.makedirs(preferred, exist_ok=True)
        probe = os.path.join(preferred, f".probe{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return preferred
    except OSError:
        tag = hashlib.sha256(HERE.encode()).hexdigest()[:12]
        fallback = os.path.join(tempfile.gettempdir(), f"xrt_b200_build_{os.getuid()}_{tag}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def library_path() -> str:
    return os.path.join(build_dir(), LIB_NAME)


def is_current() -> bool:
    out = build_dir()
    stamp = os.path.join(out, "stamp.txt")
    if not (os.path.exists(os.path.join(out, LIB_NAME)) and os.path.exists(stamp)):
        return False
    with open(stamp) as fh:
        return fh.read().strip() == _source_hash()


def _compile_one(nvcc: str, name: str, out: str, extra: list[str]) -> tuple[str, float, str]:
    start = time.time()
    obj = os.path.join(out, name[:-3] + ".o")
    cmd = [nvcc] + NVCC_FLAGS + extra + ["-I", HERE, "-c", os.path.join(HERE, name), "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise KernelError(f"nvcc failed on {name}:\n{proc.stdout}\n{proc.stderr}")
    return obj, time.time() - start, proc.stderr


def build(force: bool = False, verbose_ptxas: bool = False) -> str:
    """Compiles what is needed and returns the path of the shared library."""
    out = build_dir()
    lib = os.path.join(out, LIB_NAME)
    if not force and is_current():
        return lib
    nvcc = find_nvcc()
    names = sources()
    _say(f"compiling {len(names)} CUDA files for sm_100a into {out}")
    extra = ["-Xptxas", "-v"] if verbose_ptxas else []
    objects = []
    workers = max(1, min(len(names), os.cpu_count() or 1))
    with concurrent.futures.ThreadPoolExecutor(workers) as pool:
        futures = {pool.submit(_compile_one, nvcc, n, out, extra): n for n in names}
        done = 0
        for fut in concurrent.futures.as_completed(futures):
            obj, seconds, stderr = fut.result()
            done += 1
            _say(f"  [{done}/{len(names)}] {futures[fut]} ({seconds:.1f} s)")
            if verbose_ptxas and stderr:
                print(stderr, file=sys.stderr)
            objects.append(obj)
    tmp_lib = lib + f".tmp{os.getpid()}"
    link = [nvcc, "-shared", "-o", tmp_lib] + sorted(objects) + LINK_LIBS
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise KernelError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, lib)
    with open(os.path.join(out, "stamp.txt"), "w") as fh:
        fh.write(_source_hash())
    _say(f"built {lib}")
    return lib


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose_ptxas="--ptxas" in sys.argv)
