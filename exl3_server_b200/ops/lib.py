"""Building and loading the kernel library (``libexl3b200.so``).

The kernels are plain CUDA C++ with C entry points; they are compiled for
sm_100a with nvcc and loaded with ctypes.  Nothing is compiled at import time:
the first call of ``library()`` compiles what is missing or stale (sources are
hashed), prints a line per file and a line every few seconds while it waits,
and keeps the result in ``csrc/_build`` inside the package, or in a per-user
temporary folder when the package folder cannot be written.  There is no
fallback: without the library every kernel call raises.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libexl3b200.so"
NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
ABI_VERSION = 5


class KernelLibraryError(RuntimeError):
    """The kernel library is missing and cannot be built, or a kernel failed."""


_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()


def _say(msg: str) -> None:
    print(f"[exl3_server_b200] {msg}", file=sys.stderr, flush=True)


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(paths: List[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in paths:
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _find_nvcc() -> Optional[str]:
    for cand in (os.environ.get("EXL3_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    return None


def _build_dir() -> str:
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"exl3_server_b200-{os.getuid()}", "_build")
        os.makedirs(d, exist_ok=True)
        return d


def _compile_one(nvcc: str, src: str, obj: str) -> None:
    t0 = time.time()
    cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelLibraryError(f"nvcc failed on {os.path.basename(src)}:\n{r.stdout}\n{r.stderr}")
    _say(f"compiled {os.path.basename(src)} in {time.time() - t0:.1f}s")


def build(verbose: bool = True) -> str:
    """Compiles the library if it is missing or older than its sources and
    returns its path."""
    out_dir = _build_dir()
    lib_path = os.path.join(out_dir, LIB_NAME)
    stamp_path = os.path.join(out_dir, "build.json")
    srcs = sources()
    heads = _headers()
    head_digest = _digest(heads)
    with open(os.path.join(out_dir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            stamp = {}
            if os.path.exists(stamp_path):
                try:
                    with open(stamp_path) as f:
                        stamp = json.load(f)
                except (OSError, ValueError):
                    stamp = {}
            want = {os.path.basename(s): _digest([s]) + head_digest for s in srcs}
            have = stamp.get("objects", {})
            todo = [s for s in srcs if have.get(os.path.basename(s)) != want[os.path.basename(s)]
                    or not os.path.exists(os.path.join(out_dir, os.path.basename(s) + ".o"))]
            if not todo and os.path.exists(lib_path) and set(have) == set(want):
                return lib_path
            nvcc = _find_nvcc()
            if nvcc is None:
                raise KernelLibraryError(
                    "the CUDA kernel library is not built and nvcc was not found "
                    "(looked at $EXL3_NVCC, $CUDA_HOME/bin, PATH and /usr/local/cuda/bin)")
            _say(f"compiling {len(todo)} CUDA source file(s) for sm_100a into {out_dir} (first call only)")
            done = threading.Event()

            def ticker() -> None:
                t0 = time.time()
                while not done.wait(10.0):
                    _say(f"still compiling ... {time.time() - t0:.0f}s")

            th = threading.Thread(target=ticker, daemon=True)
            th.start()
            try:
                with ThreadPoolExecutor(max_workers=max(1, min(len(todo), os.cpu_count() or 2))) as pool:
                    futs = [pool.submit(_compile_one, nvcc, s, os.path.join(out_dir, os.path.basename(s) + ".o"))
                            for s in todo]
                    for f in futs:
                        f.result()
                objs = [os.path.join(out_dir, os.path.basename(s) + ".o") for s in srcs]
                tmp = lib_path + f".tmp{os.getpid()}"
                r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-gencode",
                                    "arch=compute_100a,code=sm_100a"], capture_output=True, text=True)
                if r.returncode != 0:
                    raise KernelLibraryError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
                os.replace(tmp, lib_path)
            finally:
                done.set()
            with open(stamp_path, "w") as f:
                json.dump({"objects": want}, f)
            _say(f"built {lib_path}")
            return lib_path
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def library() -> ctypes.CDLL:
    """The loaded kernel library; builds it on the first call."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelLibraryError(f"cannot load {path}: {e}")
            lib.exl3_last_error.restype = ctypes.c_char_p
            lib.exl3_abi_version.restype = ctypes.c_int
            if lib.exl3_abi_version() != ABI_VERSION:
                raise KernelLibraryError(f"{path} has ABI {lib.exl3_abi_version()}, expected {ABI_VERSION}")
            _lib = lib
    return _lib


def library_path() -> str:
    return os.path.join(_build_dir(), LIB_NAME)
