"""Builds and loads the sm_100a kernel library.

The kernels are plain CUDA with a C ABI (no torch headers), compiled by ``nvcc`` for
``compute_100a/sm_100a`` into one shared library next to the sources
(``csrc/_build/libgophonic_b200.so``) and opened with ``ctypes``.  The library is rebuilt when a
source or a flag changes (a digest of both is stored beside it).  Where the package folder
cannot be written, the build goes to a per-user folder under the system's temporary directory.
While compiling, a line is printed every few seconds so a first call does not look hung.

There is no fallback: if the library cannot be built or loaded, importing the kernel
operations raises.

With ``GOPHONIC_B200_CHECKED=1`` in the environment a second library is built and loaded instead,
compiled with ``-DGB_CHECKED``: every index its kernels take into the block table, a cache plane,
the embedding table or a token source is held against its bound first, and an index out of bounds
is recorded (``ops.checked_status()``) and not used.  It is the stand-in for a memory checker where
none can be run, and costs a few per cent.
"""
from __future__ import annotations

import concurrent.futures
import ctypes
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libgophonic_b200.so"
CHECKED_LIB_NAME = "libgophonic_b200_checked.so"
CHECKED_FLAG = "-DGB_CHECKED"

SOURCES = [
    "elementwise.cu",
    "cache_fill.cu",
    "gemm_simt.cu",
    "gemm_skinny.cu",
    "gemm_skinny_fold.cu",
    "gemm_tc5.cu",
    "gemm_tc5_decode.cu",
    "attention_simt.cu",
    "attention_mma.cu",
    "attention_tc5.cu",
    "sampling.cu",
    "no_alloc.cu",
    "dispatch.cu",
]
HEADERS = ["common.cuh", "mma.cuh", "tc5.cuh", "no_alloc.h", "api.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def _existing(names: List[str]) -> List[str]:
    return [n for n in names if os.path.exists(os.path.join(HERE, n))]


def _nvcc() -> str:
    cand = [os.environ.get("GOPHONIC_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for c in cand:
        if c and os.path.exists(c):
            return c
    raise BuildError("the CUDA kernel library has to be compiled and nvcc was not found "
                     "(looked at $GOPHONIC_B200_NVCC, PATH and /usr/local/cuda/bin/nvcc)")


def checked_requested() -> bool:
    return os.environ.get("GOPHONIC_B200_CHECKED", "") not in ("", "0")


def _digest(flags: Optional[List[str]] = None) -> str:
    h = hashlib.sha256()
    for name in _existing(SOURCES) + _existing(HEADERS):
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + (flags or [])).encode())
    return h.hexdigest()


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe_{os.getpid()}")
        with open(probe, "w") as f:
            f.write("x")
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    override = os.environ.get("GOPHONIC_B200_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    in_tree = os.path.join(HERE, "_build")
    if _writable_dir(in_tree):
        return in_tree
    fallback = os.path.join(tempfile.gettempdir(), f"gophonic_b200_build_{os.getuid()}")
    if _writable_dir(fallback):
        return fallback
    raise BuildError(f"neither {in_tree} nor {fallback} can be written; set GOPHONIC_B200_BUILD_DIR")


def _up_to_date(bdir: str, digest: str, lib_name: str = LIB_NAME) -> bool:
    lib = os.path.join(bdir, lib_name)
    stamp = os.path.join(bdir, lib_name + ".stamp.json" if lib_name != LIB_NAME else "stamp.json")
    if not (os.path.exists(lib) and os.path.exists(stamp)):
        return False
    try:
        with open(stamp) as f:
            return json.load(f).get("digest") == digest
    except (OSError, ValueError):
        return False


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[gophonic_b200] {msg}", file=sys.stderr, flush=True)


def ensure_built(verbose: bool = True, extra_flags: Optional[List[str]] = None, checked: bool = False) -> str:
    """Compile the library if it is missing or stale; return its path.  ``checked``: the library with
    bounds-checked indices, kept beside the ordinary one."""
    extra = list(extra_flags or []) + ([CHECKED_FLAG] if checked else [])
    lib_name = CHECKED_LIB_NAME if checked else LIB_NAME
    stamp_name = lib_name + ".stamp.json" if checked else "stamp.json"
    digest = _digest(extra)
    # an up-to-date library anywhere we would build is used as it is
    in_tree = os.path.join(HERE, "_build")
    if not os.environ.get("GOPHONIC_B200_BUILD_DIR") and _up_to_date(in_tree, digest, lib_name):
        return os.path.join(in_tree, lib_name)
    bdir = build_dir()
    if _up_to_date(bdir, digest, lib_name):
        return os.path.join(bdir, lib_name)
    nvcc = _nvcc()
    sources = _existing(SOURCES)
    flags = NVCC_FLAGS + extra
    _say(f"compiling {len(sources)} CUDA sources for sm_100a into {bdir} (first call only"
         f"{'; the build with checked indices' if checked else ''})", verbose)
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s", verbose)

    tick = threading.Thread(target=ticker, daemon=True)
    tick.start()
    tag = f"{os.getpid()}"

    def compile_one(src: str) -> str:
        obj = os.path.join(bdir, src.replace(".cu", f".{tag}.o"))
        cmd = [nvcc] + flags + ["-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise BuildError(f"nvcc failed on {src}:\n{r.stdout}")
        _say(f"compiled {src} ({time.time() - t0:.0f} s)", verbose)
        return obj

    objs: List[str] = []
    try:
        workers = max(1, min(len(sources), os.cpu_count() or 1))
        with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as ex:
            objs = list(ex.map(compile_one, sources))
        tmp_lib = os.path.join(bdir, f"{lib_name}.{tag}.tmp")
        cmd = [nvcc, "-shared", "-o", tmp_lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise BuildError(f"linking the kernel library failed:\n{r.stdout}")
        os.replace(tmp_lib, os.path.join(bdir, lib_name))
        with open(os.path.join(bdir, stamp_name), "w") as f:
            json.dump({"digest": digest, "flags": flags, "sources": sources}, f)
    finally:
        done.set()
        # this build's objects, also those of sources that compiled before another one failed
        for name in os.listdir(bdir):
            if name.endswith(f".{tag}.o") or name.endswith(f".{tag}.tmp"):
                try:
                    os.remove(os.path.join(bdir, name))
                except OSError:
                    pass
    _say(f"kernel library ready after {time.time() - t0:.0f} s", verbose)
    return os.path.join(bdir, lib_name)


_lib: Optional[ctypes.CDLL] = None
_lib_lock = threading.Lock()


def load(verbose: bool = True) -> ctypes.CDLL:
    """The loaded library (built on first use)."""
    global _lib
    with _lib_lock:
        if _lib is None:
            path = ensure_built(verbose=verbose, checked=checked_requested())
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from e
            _lib.gb_last_error.restype = ctypes.c_char_p
        return _lib


def library_file() -> Optional[str]:
    return _lib._name if _lib is not None else None


if __name__ == "__main__":
    print(ensure_built(verbose=True))
