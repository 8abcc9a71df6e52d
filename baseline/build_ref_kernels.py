#!/usr/bin/env python3
"""Compiles the reference's own Qwen3-path CUDA kernels, unmodified, for sm_100a into one shared object, so that
``bench_kernels.py --impl reference`` can time them beside this package's kernels on the same GPU.

    python baseline/build_ref_kernels.py /path/to/rayze-ai/dinfer     ->  baseline/_ref/libdinfer_ref_kernels.so

The reference is a Rust workspace and cannot be built whole without cargo, but its kernels are plain CUDA with a C
ABI (crates/kernels/cuda/kernels.h) and no dependency beyond the toolkit.  The files and flags are those of its own
build (crates/kernels/build.rs:120-146: ``nvcc -c -std=c++17 -O3 --expt-relaxed-constexpr -Xcompiler -fPIC -I cuda``
with ``CUDA_ARCHS=100`` -> ``compute_100a``), limited to the kernels the Qwen3 model runs: norms, activation and
embedding, q/k post-processing, attention (prefill, paged, decode v1/v2/v3), the small-M products and sampling.
Its ``*_sm100.cu`` files serve other architectures and are left out (their device-side waits are unbounded), so
``MEGA_SM100`` stays undefined, as in a build without them.  Nothing is copied into this repository: the sources
are read where the reference lies and only the built library is kept (under the git-ignored ``baseline/_ref``).
"""
import os
import subprocess
import sys

FILES = ["norm.cu", "activation.cu", "qkv_post.cu", "gqa.cu", "gqa_decode_v3.cu", "gemm_small_m.cu", "sampling.cu"]
HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "libdinfer_ref_kernels.so")


def main(ref_root: str) -> int:
    cuda = os.path.join(ref_root, "crates", "kernels", "cuda")
    missing = [f for f in FILES if not os.path.isfile(os.path.join(cuda, f))]
    if missing:
        print(f"not found under {cuda}: {missing}", file=sys.stderr)
        return 1
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, "-std=c++17", "-O3", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-I", cuda,
           "-gencode=arch=compute_100a,code=sm_100a", "-shared", "-o", OUT] + [os.path.join(cuda, f) for f in FILES]
    print(" ".join(cmd), flush=True)
    rc = subprocess.call(cmd, cwd=cuda)
    if rc == 0:
        print("built", OUT)
    return rc


if __name__ == "__main__":
    sys.exit(main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference"))
