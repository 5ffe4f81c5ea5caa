"""Stages the reference's own Python package and tests next to the libraries built for it.

TEST INFRASTRUCTURE ONLY. The reference's Python layer (python/src/loom_kernels)
finds its compiled dispatcher the way its loader says
(python/src/loom_kernels/_torch_extension.py:90-110): from a source checkout it
looks for ``<root>/build/libloom_kernels_torch.so``, where ``<root>`` is the
first parent directory holding ``Cargo.toml`` and ``crates/loom-cuda-bridge``.
This script lays such a root out under ``oracle/_ref/checkout`` (git-ignored,
never committed): the reference's package and its two hot-path test files as
they are, the dispatcher built by ``build_reference_dispatcher.py`` and this
tree's ``libloom_cuda_bridge.so`` under ``build/``. A GPU test then runs the
reference's own pytest files against this library
(``tests/test_gpu_reference_python_tests.py``).

Usage:  python oracle/stage_reference_python.py
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle.reference_root import reference_root  # noqa: E402

CHECKOUT = os.path.join(HERE, "_ref", "checkout")
TEST_FILES = ("test_paged_decode_attention.py", "test_rope_paged_kv.py")


def stage(root: str | None = None) -> str | None:
    """Returns the staged root, or None when there is no reference checkout or dispatcher."""
    root = root or reference_root()
    dispatcher = os.path.join(HERE, "_ref", "libloom_kernels_torch.so")
    bridge = os.path.join(ROOT, "attnarc_b200", "libloom_cuda_bridge.so")
    if root is None or not os.path.exists(dispatcher) or not os.path.exists(bridge):
        return None
    package = os.path.join(root, "python", "src", "loom_kernels")
    tests = os.path.join(root, "python", "tests")
    if not os.path.isdir(package) or not all(os.path.exists(os.path.join(tests, name)) for name in TEST_FILES):
        return None
    if os.path.isdir(CHECKOUT):
        shutil.rmtree(CHECKOUT)
    os.makedirs(os.path.join(CHECKOUT, "crates", "loom-cuda-bridge"))
    os.makedirs(os.path.join(CHECKOUT, "build"))
    os.makedirs(os.path.join(CHECKOUT, "python", "tests"))
    with open(os.path.join(CHECKOUT, "Cargo.toml"), "w") as marker:
        marker.write("# marker: lets the staged Python package find build/ the way a source checkout does\n")
    shutil.copytree(package, os.path.join(CHECKOUT, "python", "src", "loom_kernels"),
                    ignore=shutil.ignore_patterns("__pycache__", "lib"))
    for name in TEST_FILES:
        shutil.copy(os.path.join(tests, name), os.path.join(CHECKOUT, "python", "tests", name))
    shutil.copy(dispatcher, os.path.join(CHECKOUT, "build", "libloom_kernels_torch.so"))
    return CHECKOUT


if __name__ == "__main__":
    print(stage() or "nothing staged: no reference checkout, or the dispatcher has not been built")
