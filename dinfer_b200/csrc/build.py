"""Builds the kernel libraries for sm_100a with nvcc: one shared object per ``.cu`` file.

A library is compiled at the first call that needs it (so a model compiles only what it uses)
and kept under ``csrc/_build/`` inside the package; when that folder cannot be written, under a
per-user folder in the temporary directory.  A stamp of the source texts and flags in the file
name makes a changed source compile again.  No torch headers are involved: the libraries have a
C ABI and are loaded with ctypes.  The reference builds the same way, one ``nvcc -c`` per ``.cu``
from ``crates/kernels/build.rs:37-146``.
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
from typing import Dict, Iterable, List

CSRC = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fvisibility=hidden"]

# library name -> (source file, extra link flags)
LIBRARIES: Dict[str, tuple] = {
    "norm": ("norm.cu", []),
    "elementwise": ("elementwise.cu", []),
    "qk_post": ("qk_post.cu", []),
    "attention_generic": ("attention_generic.cu", []),
    "gemm_f32": ("gemm_f32.cu", []),
    "sampling": ("sampling.cu", []),
    "attention_tc": ("attention_tc.cu", []),
    "attention_decode": ("attention_decode.cu", []),
    "gemm_tc": ("gemm_tc.cu", []),
    "attention_umma": ("attention_umma.cu", []),
    "attention_umma64": ("attention_umma64.cu", []),
    # host-side bookkeeping (page pools, cache manager, decode plans): plain C++, no CUDA
    "host_core": ("host_core.cpp", []),
}
CXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    cands = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            cands.append(os.path.join(os.environ[var], "bin", "nvcc"))
    cands.append("/usr/local/cuda/bin/nvcc")
    w = shutil.which("nvcc")
    if w:
        cands.append(w)
    for c in cands:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                     "the CUDA kernels of dinfer_b200 cannot be built")


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _stamp(source: str, extra: Iterable[str]) -> str:
    h = hashlib.sha256()
    for fn in [source] + _headers():
        with open(os.path.join(CSRC, fn), "rb") as f:
            h.update(fn.encode())
            h.update(f.read())
    flags = CXX_FLAGS if source.endswith(".cpp") else ARCH_FLAGS + NVCC_FLAGS
    h.update(" ".join(flags + list(extra)).encode())
    return h.hexdigest()[:12]


_build_dir_cache = None


def build_dir() -> str:
    global _build_dir_cache
    if _build_dir_cache:
        return _build_dir_cache
    cands = [os.path.join(CSRC, "_build"),
             os.path.join(tempfile.gettempdir(), f"dinfer_b200_build_{os.getuid()}")]
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            _build_dir_cache = d
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {cands}")


def library_path(name: str) -> str:
    source, extra = LIBRARIES[name]
    return os.path.join(build_dir(), f"libdinfer_{name}_{_stamp(source, extra)}.so")


def _compile(name: str, verbose: bool) -> str:
    source, extra = LIBRARIES[name]
    out = library_path(name)
    if os.path.isfile(out):
        return out
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    if source.endswith(".cpp"):
        cxx = shutil.which(os.environ.get("CXX", "g++")) or shutil.which("c++")
        if not cxx:
            raise BuildError("no C++ compiler found (g++ or $CXX); the host core of dinfer_b200 cannot be built")
        cmd = [cxx] + CXX_FLAGS + ["-I", CSRC, "-o", tmp, os.path.join(CSRC, source)] + list(extra)
    else:
        cmd = [find_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + ["-I", CSRC, "-o", tmp, os.path.join(CSRC, source)] + list(extra)
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"the compiler failed on {source}:\n{' '.join(cmd)}\n{proc.stdout}")
    os.replace(tmp, out)
    # drop older builds of the same library
    prefix = f"libdinfer_{name}_"
    for fn in os.listdir(os.path.dirname(out)):
        if fn.startswith(prefix) and fn.endswith(".so") and fn != os.path.basename(out):
            try:
                os.remove(os.path.join(os.path.dirname(out), fn))
            except OSError:
                pass
    if verbose:
        print(f"[dinfer_b200] built {name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def ensure_built(names: Iterable[str], verbose: bool = True) -> Dict[str, str]:
    """Compile the named libraries that are missing (in parallel) and return their paths.
    While nvcc runs, a line is printed every few seconds."""
    names = list(dict.fromkeys(names))
    for n in names:
        if n not in LIBRARIES:
            raise BuildError(f"unknown kernel library {n!r}")
    missing = [n for n in names if not os.path.isfile(library_path(n))]
    if missing:
        if verbose:
            cuda = [n for n in missing if not LIBRARIES[n][0].endswith(".cpp")]
            host = [n for n in missing if LIBRARIES[n][0].endswith(".cpp")]
            what = "; ".join(x for x in ((f"CUDA kernels for sm_100a: {', '.join(cuda)}" if cuda else ""),
                                         (f"host code: {', '.join(host)}" if host else "")) if x)
            print(f"[dinfer_b200] compiling {what}", file=sys.stderr, flush=True)
        t0 = time.time()
        with ThreadPoolExecutor(max_workers=min(len(missing), os.cpu_count() or 4)) as pool:
            futs = {n: pool.submit(_compile, n, verbose) for n in missing}
            while True:
                pending = [n for n, f in futs.items() if not f.done()]
                if not pending:
                    break
                time.sleep(0.5)
                if verbose and int(time.time() - t0) % 5 == 0 and (time.time() - t0) % 1 < 0.5:
                    print(f"[dinfer_b200] still compiling ({int(time.time() - t0)} s): "
                          f"{', '.join(pending)}", file=sys.stderr, flush=True)
            for f in futs.values():
                f.result()
    return {n: library_path(n) for n in names}


def build_all(verbose: bool = True) -> Dict[str, str]:
    return ensure_built(list(LIBRARIES), verbose)


if __name__ == "__main__":
    for k, v in build_all().items():
        print(k, v)
