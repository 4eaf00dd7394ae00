"""Compiles the CUDA sources of this folder for sm_100a and loads them as one shared library.

The library is plain C ABI (``extern "C"`` launchers over raw device pointers and a stream),
built with ``nvcc`` alone and opened with ``ctypes``.  Objects and the library live in
``lily_b200/csrc/_build`` and are named by a hash of their source text and the compiler flags,
so a changed source is rebuilt and a stale binary is never loaded.  When that folder cannot
be written (a read-only checkout) a per-user folder under the temporary directory is used.

The first call in a fresh checkout compiles (a line is printed as each file starts and ends);
there is no fallback: without ``nvcc`` or without the library every kernel call raises.

Plays the role of lily/layers/quantization/cuda_ops.py:27-65 (JIT build of lily/csrc), except
that a failed build there makes callers fall back to PyTorch and here it is an error.
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
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))

SOURCES = ["elementwise.cu", "gemm_fp32.cu", "gemm_skinny.cu", "gemm_tcgen05.cu", "attention_simt.cu", "attention_mma.cu", "attention_tcgen05.cu", "sampling.cu",
           "attention_decode_static.cu"]
HEADERS = ["common.cuh", "attention_args.cuh", "no_alloc.h"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


# extra compiler flags for experiments (e.g. -DLILY_DECODE_STAGES=3); they enter the binaries' names
NVCC_FLAGS += os.environ.get("LILY_B200_NVCC_FLAGS", "").split()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[lily_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("LILY_B200_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $LILY_B200_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                     "the CUDA kernels of lily_b200 cannot be built and there is no fallback")


def _digest(paths: List[str], extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(os.path.basename(p).encode())     # not the folder: a copied checkout reuses its binaries
            h.update(f.read())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    want = os.environ.get("LILY_B200_BUILD_DIR") or os.path.join(HERE, "_build")
    try:
        os.makedirs(want, exist_ok=True)
        probe = os.path.join(want, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return want
    except OSError:
        alt = os.path.join(tempfile.gettempdir(), f"lily_b200_build_{os.getuid()}")
        os.makedirs(alt, exist_ok=True)
        return alt


def _run(cmd: List[str], what: str) -> None:
    t0 = time.time()
    _say(f"{what} ...")
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def beat():
        while not done.wait(15.0):
            _say(f"  still {what} ({time.time() - t0:.0f} s)")
    t = threading.Thread(target=beat, daemon=True)
    t.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"{what} failed (exit {proc.returncode}):\n{' '.join(cmd)}\n{out}")
    _say(f"{what} done in {time.time() - t0:.1f} s")


def library_path(build_dir: Optional[str] = None) -> str:
    srcs = [os.path.join(HERE, s) for s in SOURCES + HEADERS]
    tag = _digest(srcs, " ".join(NVCC_FLAGS))
    return os.path.join(build_dir or _build_dir(), f"liblily_b200_{tag}.so")


def build(verbose: bool = True) -> str:
    """Compiles what is missing and returns the path of the shared library."""
    bdir = _build_dir()
    lib = library_path(bdir)
    if os.path.isfile(lib):
        return lib
    nvcc = find_nvcc()
    headers = [os.path.join(HERE, h) for h in HEADERS]
    objects, jobs = [], []
    for s in SOURCES:
        src = os.path.join(HERE, s)
        obj = os.path.join(bdir, f"{os.path.splitext(s)[0]}_{_digest([src] + headers, ' '.join(NVCC_FLAGS))}.o")
        objects.append(obj)
        if not os.path.isfile(obj):
            jobs.append((src, obj))
    if jobs:
        _say(f"compiling {len(jobs)} CUDA source file(s) for sm_100a into {bdir}")

        def compile_one(job):
            src, obj = job
            tmp = f"{obj}.{os.getpid()}.tmp"
            _run([nvcc, *NVCC_FLAGS, "-I", HERE, "-c", src, "-o", tmp], f"compiling {os.path.basename(src)}")
            os.replace(tmp, obj)
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(compile_one, jobs))
    tmp = f"{lib}.{os.getpid()}.tmp"
    _run([nvcc, "-shared", "-o", tmp, *objects], "linking")
    os.replace(tmp, lib)
    return lib


_LIB: Optional[ctypes.CDLL] = None
_LOCK = threading.Lock()


def load() -> ctypes.CDLL:
    """The loaded library; built first when needed."""
    global _LIB
    with _LOCK:
        if _LIB is None:
            _LIB = ctypes.CDLL(build())
            _LIB.lily_last_error.restype = ctypes.c_char_p
        return _LIB
