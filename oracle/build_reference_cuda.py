"""Compiles the reference's own CUDA kernels of the hot path for sm_100a.

TEST AND BASELINE INFRASTRUCTURE ONLY. The reference's GPU implementation of
the path is three plain CUDA files behind the launch ABI of ``loom_cuda.h``
(crates/loom-cuda-sys/cuda/src/paged_decode_attention.cu, rope_paged_kv.cu, and
rms_norm.cu for ``loom_cuda_status_string``). They are compiled here with nvcc
from where they lie in a reference checkout; nothing is copied, and the only
output is ``oracle/_ref/libloom_cuda_reference.so`` (git-ignored). The GPU
tests use it as a second checker (the reference's real GPU results, contexts up
to its 1024-token limit) and ``bench.py --workload cfg2-1024`` times it beside
this library. Without a reference checkout nothing is built and both are
skipped.

Usage:  python oracle/build_reference_cuda.py [reference root]   (default: $LOOM_REFERENCE_ROOT, else ../reference beside this repository)
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUTPUT_DIR = os.path.join(HERE, "_ref")
OUTPUT = os.path.join(OUTPUT_DIR, "libloom_cuda_reference.so")
SOURCES = ("paged_decode_attention.cu", "rope_paged_kv.cu", "rms_norm.cu")


def build(reference_root: str | None = None, verbose: bool = False) -> str | None:
    """Returns the path of the built library, or None if there is no reference checkout."""
    from oracle.reference_root import reference_root as locate

    reference_root = reference_root or locate()
    if reference_root is None:
        return OUTPUT if os.path.exists(OUTPUT) else None
    cuda_dir = os.path.join(reference_root, "crates", "loom-cuda-sys", "cuda")
    sources = [os.path.join(cuda_dir, "src", name) for name in SOURCES]
    if not all(os.path.exists(path) for path in sources):
        return None
    if os.path.exists(OUTPUT) and all(os.path.getmtime(p) <= os.path.getmtime(OUTPUT) for p in sources):
        return OUTPUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUTPUT_DIR, exist_ok=True)
    command = [nvcc, "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-gencode",
               "arch=compute_100a,code=sm_100a", f"-I{os.path.join(cuda_dir, 'include')}", *sources, "-o", OUTPUT]
    done = subprocess.run(command, capture_output=True, text=True)
    if verbose or done.returncode != 0:
        sys.stderr.write(done.stdout + done.stderr)
    if done.returncode != 0:
        raise RuntimeError("the reference CUDA kernels did not compile")
    return OUTPUT


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(HERE))
    result = build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True)
    print(result if result else "no reference checkout: nothing built")
