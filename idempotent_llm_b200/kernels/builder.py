"""Compiling and loading the CUDA libraries, one per storage dtype.

Sources under ``csrc/`` are compiled with nvcc for sm_100a into
``_build/<dtype>/libidm_<dtype>.so`` inside the package (or, if the package folder
cannot be written, under ``$IDM_BUILD_DIR`` or the temporary folder).  A stamp
made of the sources' and flags' hash decides whether the library is current; a
first call in a fresh checkout compiles what the requested dtype needs and
prints a line per file, and a line every few seconds while a file is still
compiling.  There is no fallback: without nvcc or with a failing compile this
raises.
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
import threading
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from typing import Dict, List

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG_DIR, "csrc")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]   # never --use_fast_math

# sources per dtype: the 32-bit library carries the plain FMA matrix product,
# the bfloat16 library the tensor-core kernels
SOURCES: Dict[str, List[str]] = {
    "float32": ["runtime.cu", "elementwise.cu", "sampler.cu", "attention_generic.cu",
                "attention_decode.cu", "gemm_f32.cu"],
    "bfloat16": ["runtime.cu", "elementwise.cu", "sampler.cu", "attention_generic.cu",
                 "attention_decode.cu", "gemm_tcgen05.cu", "attention_tcgen05.cu", "step_program.cu"],
}
DEFINES = {"float32": "-DIDM_F32", "bfloat16": "-DIDM_BF16"}
_LOADED: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[idempotent_llm_b200] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("IDM_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (PATH, /usr/local/cuda/bin, $IDM_NVCC): the CUDA kernels "
                     "cannot be compiled and there is no other path")


def _build_root() -> str:
    env = os.environ.get("IDM_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    root = os.path.join(PKG_DIR, "_build")
    try:
        os.makedirs(root, exist_ok=True)
        probe = os.path.join(root, f".w{os.getpid()}")
        open(probe, "w").close()
        os.remove(probe)
        return root
    except OSError:
        root = os.path.join(tempfile.gettempdir(), f"idempotent_llm_b200-build-{os.getuid()}")
        os.makedirs(root, exist_ok=True)
        return root


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _stamp(dtype: str, extra_flags: List[str]) -> str:
    h = hashlib.sha256()
    for name in SOURCES[dtype] + _headers():
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(name.encode() + b"\0" + f.read())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + [DEFINES[dtype]] + extra_flags).encode())
    return h.hexdigest()


def _run(cmd: List[str], what: str) -> None:
    t0 = time.time()
    done = threading.Event()

    def beat():
        while not done.wait(15.0):
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")
    th = threading.Thread(target=beat, daemon=True)
    th.start()
    try:
        p = subprocess.run(cmd, capture_output=True, text=True)
    finally:
        done.set()
    if p.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n{' '.join(cmd)}\n{p.stdout}\n{p.stderr}")


def build(dtype: str, verbose: bool = True, extra_flags: List[str] = ()) -> str:
    """Compile the library for ``dtype`` if it is not current; returns its path."""
    if dtype not in SOURCES:
        raise BuildError(f"no kernels for dtype {dtype!r}; known: {sorted(SOURCES)}")
    extra_flags = list(extra_flags) + os.environ.get("IDM_EXTRA_NVCC_FLAGS", "").split()
    out_dir = os.path.join(_build_root(), dtype)
    os.makedirs(out_dir, exist_ok=True)
    lib = os.path.join(out_dir, f"libidm_{dtype}.so")
    stamp_file = os.path.join(out_dir, "stamp")
    stamp = _stamp(dtype, extra_flags)
    with open(os.path.join(out_dir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if os.path.isfile(lib) and os.path.isfile(stamp_file) and open(stamp_file).read() == stamp:
                return lib
            nvcc = _nvcc()
            srcs = SOURCES[dtype]
            if verbose:
                _say(f"compiling {len(srcs)} CUDA files for sm_100a ({dtype}) into {out_dir}")
            t0 = time.time()
            objs = []

            def one(src):
                obj = os.path.join(out_dir, src.replace(".cu", ".o"))
                _run([nvcc, *ARCH_FLAGS, *COMMON_FLAGS, DEFINES[dtype], *extra_flags, "-I", CSRC, "-c",
                      os.path.join(CSRC, src), "-o", obj], f"{src} ({dtype})")
                return src, obj

            with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
                futs = [ex.submit(one, s) for s in srcs]
                for n, f in enumerate(as_completed(futs), 1):
                    src, obj = f.result()
                    objs.append(obj)
                    if verbose:
                        _say(f"  [{n}/{len(srcs)}] {src} ({time.time() - t0:.0f} s)")
            tmp = lib + f".tmp{os.getpid()}"
            _run([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *sorted(objs), "-lcuda"], f"link ({dtype})")
            os.replace(tmp, lib)
            with open(stamp_file, "w") as f:
                f.write(stamp)
            if verbose:
                _say(f"built {os.path.basename(lib)} in {time.time() - t0:.0f} s")
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def load(dtype: str) -> ctypes.CDLL:
    """The compiled library for ``dtype`` (built at the first call)."""
    lib = _LOADED.get(dtype)
    if lib is None:
        path = build(dtype)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"{path} was built but cannot be loaded: {e}") from None
        lib.idm_last_error.restype = ctypes.c_char_p
        lib.idm_dtype_name.restype = ctypes.c_char_p
        if lib.idm_dtype_name().decode() != dtype:
            raise BuildError(f"{path} was compiled for {lib.idm_dtype_name().decode()}, not {dtype}")
        _LOADED[dtype] = lib
    return lib
