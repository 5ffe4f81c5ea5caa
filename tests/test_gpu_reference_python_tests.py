"""The reference's OWN Python tests, unmodified, run against this library.

``oracle/stage_reference_python.py`` lays out the reference's Python package
(python/src/loom_kernels), its hot-path test files (python/tests/
test_paged_decode_attention.py, test_rope_paged_kv.py) and its dispatcher
compiled against ``libloom_cuda_bridge.so`` as the package's own loader expects
(python/src/loom_kernels/_torch_extension.py:90-110). Here pytest runs those
files in a child process; every collected test must pass. The cases of
test_rope_paged_kv.py that compare with vLLM's ``_C`` operators are left out
(they need the vLLM build the reference was qualified with); its schema,
launch-counter, argument-rejection, torch.compile, CUDA-graph and
external-stream cases run. Skipped where nothing was staged (no reference
checkout on the machine that built the tree).
"""

import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKOUT = os.path.join(ROOT, "oracle", "_ref", "checkout")


def run_reference_tests(test_file, *pytest_args):
    if not os.path.exists(os.path.join(CHECKOUT, "build", "libloom_kernels_torch.so")):
        pytest.skip("the reference's Python package was not staged")
    environment = dict(os.environ)
    environment["PYTHONPATH"] = os.path.join(CHECKOUT, "python", "src")
    # the dispatcher's libloom_cuda_bridge.so is this tree's
    environment["LD_LIBRARY_PATH"] = os.pathsep.join(
        [os.path.join(ROOT, "attnarc_b200"), environment.get("LD_LIBRARY_PATH", "")])
    command = [sys.executable, "-m", "pytest", os.path.join(CHECKOUT, "python", "tests", test_file), "-q",
               "-p", "no:cacheprovider", "--rootdir", os.path.join(CHECKOUT, "python"), *pytest_args]
    done = subprocess.run(command, capture_output=True, text=True, cwd=os.path.join(CHECKOUT, "python"),
                          env=environment, timeout=1500)
    tail = (done.stdout + done.stderr)[-4000:]
    summary = re.search(r"(\d+) passed", done.stdout)
    print(f"reference {test_file}: {done.stdout.strip().splitlines()[-1] if done.stdout.strip() else 'no output'}")
    assert done.returncode == 0, tail
    assert summary and int(summary.group(1)) > 0, tail
    assert " failed" not in done.stdout.splitlines()[-1], tail
    return int(summary.group(1))


def test_reference_paged_decode_attention_tests_pass():
    # 13 shapes x 3 dtypes against its PyTorch oracle, vLLM's interleaved stride, external stream,
    # opcheck + torch.compile, telemetry and error text, the support predicate
    assert run_reference_tests("test_paged_decode_attention.py") >= 40


def test_reference_rope_paged_kv_tests_pass():
    passed = run_reference_tests("test_rope_paged_kv.py", "-k", "not matches_vllm and not packed_qkv")
    assert passed >= 7
