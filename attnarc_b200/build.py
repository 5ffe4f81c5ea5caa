"""Builds ``libloom_cuda_bridge.so`` in-tree with nvcc for sm_100a.

The library holds the CUDA kernels, the launch ABI (``include/loom_launch.h``),
the safe dispatch layer and the checked bridge ABI (``include/loom_bridge.h``).
It is compiled here rather than through a JIT cache so that the built file
travels with the source tree. Run ``python -m attnarc_b200.build``; extra nvcc
flags (``-DLOOM_FP8_KEY_BY_ALU=1`` ...) are taken from ``LOOM_NVCC_FLAGS``.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
SOURCE_DIR = os.path.join(PACKAGE_DIR, "csrc")
BUILD_DIR = os.path.join(PACKAGE_DIR, "build")
LIBRARY = os.path.join(PACKAGE_DIR, "libloom_cuda_bridge.so")

SOURCES = [
    "rope_paged_kv_sm100.cu",
    "paged_decode_sm100.cu",
    "kv_block_move_sm100.cu",
    "multi_token_sm100.cu",
    "peer_exchange_sm100.cu",
    "dispatch.cpp",
    "bridge.cpp",
    "partition.cpp",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-Wall,-Wextra",
    "-Xptxas", "-v",
]


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return found


def _headers() -> list[str]:
    include_dir = os.path.join(os.path.dirname(PACKAGE_DIR), "include")
    out = [os.path.join(SOURCE_DIR, n) for n in os.listdir(SOURCE_DIR) if n.endswith((".hpp", ".cuh", ".h"))]
    out += [os.path.join(include_dir, n) for n in os.listdir(include_dir)]
    return out


def _stale(target: str, inputs: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    built = os.path.getmtime(target)
    return any(os.path.getmtime(path) > built for path in inputs)


def _compile(source: str, force: bool) -> tuple[str, str]:
    path = os.path.join(SOURCE_DIR, source)
    obj = os.path.join(BUILD_DIR, source + ".o")
    log = ""
    if force or _stale(obj, [path] + _headers()):
        extra = os.environ.get("LOOM_NVCC_FLAGS", "").split()
        cmd = [nvcc_path(), *NVCC_FLAGS, *extra, "-c", path, "-o", obj]
        done = subprocess.run(cmd, capture_output=True, text=True)
        log = done.stdout + done.stderr
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed on {source}:\n{log}")
    return obj, log


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles what changed and links the shared library; returns its path."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(lambda s: _compile(s, force), SOURCES))
    objects = [obj for obj, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if force or _stale(LIBRARY, objects):
        cmd = [nvcc_path(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC",
               # Calls between this library's own entry points bind inside it: the reference's
               # library exports the same names and may be loaded in the same process.
               "-Xlinker", "-Bsymbolic",
               "-o", LIBRARY, *objects]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError("link failed:\n" + done.stdout + done.stderr)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
