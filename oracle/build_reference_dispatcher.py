"""Compiles the reference's UNMODIFIED torch dispatcher against this bridge.

TEST INFRASTRUCTURE ONLY. The reference's PyTorch adapter is a small C++
library (python/csrc/*.cpp in the reference tree, LibTorch stable ABI) that
registers ``torch.ops.loom_kernels.*`` and calls the checked bridge ABI
(``loom_cuda_bridge.h``). It is compiled here from the sources where they lie
in the reference checkout, with the reference's own bridge header, and linked
against ``attnarc_b200/libloom_cuda_bridge.so``: if it links, every symbol the
reference's adapter needs is exported with a compatible signature, and the GPU
test ``tests/test_gpu_reference_dispatcher.py`` then drives the decode and the
RoPE/KV write through the reference's own operator registrations.

Nothing of the reference is copied: the only output is
``oracle/_ref/libloom_kernels_torch.so`` (git-ignored). Without a reference
checkout the script does nothing and the GPU test is skipped.

Usage:  python oracle/build_reference_dispatcher.py [reference root]   (default: $LOOM_REFERENCE_ROOT, else ../reference beside this repository)
"""

from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUTPUT_DIR = os.path.join(HERE, "_ref")
OUTPUT = os.path.join(OUTPUT_DIR, "libloom_kernels_torch.so")
BRIDGE_DIR = os.path.join(ROOT, "attnarc_b200")


def build(reference_root: str | None = None, verbose: bool = False) -> str | None:
    """Returns the path of the built dispatcher, or None if there is no reference checkout."""
    from oracle.reference_root import reference_root as locate

    reference_root = reference_root or locate()
    if reference_root is None:
        return OUTPUT if os.path.exists(OUTPUT) else None
    sources = sorted(glob.glob(os.path.join(reference_root, "python", "csrc", "*.cpp")))
    bridge_header_dir = os.path.join(reference_root, "crates", "loom-cuda-bridge", "include")
    if not sources or not os.path.isdir(bridge_header_dir):
        return None
    if not os.path.exists(os.path.join(BRIDGE_DIR, "libloom_cuda_bridge.so")):
        raise RuntimeError("build attnarc_b200/libloom_cuda_bridge.so first (python -m attnarc_b200.build)")
    inputs = sources + glob.glob(os.path.join(reference_root, "python", "csrc", "*.h")) + [
        os.path.join(BRIDGE_DIR, "libloom_cuda_bridge.so")]
    if os.path.exists(OUTPUT) and all(os.path.getmtime(p) <= os.path.getmtime(OUTPUT) for p in inputs):
        return OUTPUT
    from torch.utils.cpp_extension import include_paths, library_paths

    os.makedirs(OUTPUT_DIR, exist_ok=True)
    cuda_include = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    command = ["g++", "-shared", "-fPIC", "-O2", "-std=c++17", "-DUSE_CUDA", "-o", OUTPUT, *sources,
               f"-I{bridge_header_dir}", f"-I{cuda_include}"]
    command += [f"-I{path}" for path in include_paths()]
    command += [f"-L{BRIDGE_DIR}", "-lloom_cuda_bridge", f"-L{library_paths()[0]}", "-Wl,--as-needed",
                "-ltorch_cuda", "-ltorch", "-ltorch_cpu", "-lc10",
                # found next to the bridge when both travel inside the repository
                "-Wl,-rpath,$ORIGIN/../../attnarc_b200", f"-Wl,-rpath,{library_paths()[0]}"]
    done = subprocess.run(command, capture_output=True, text=True)
    if verbose or done.returncode != 0:
        sys.stderr.write(done.stdout + done.stderr)
    if done.returncode != 0:
        raise RuntimeError("the reference dispatcher did not compile or link against this bridge")
    return OUTPUT


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(HERE))
    result = build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True)
    print(result if result else "no reference checkout: nothing built")
