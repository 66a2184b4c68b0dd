"""Allocation failures injected on the host: the library reports them and stays usable.

A child process runs with `tests/alloc_fault_shim.c` preloaded, a counting
`cudaMalloc` that can be told to fail its next call with
`cudaErrorMemoryAllocation` (the approach of the reference's
`tests/cuda_fail_alloc.c` and `tests/test_cuda.py:124-226`). Nothing on the GPU
faults: the failing call never reaches the driver. Checked in the child
(`tests/alloc_faults_child.py`): scratch growth, peer-region allocation and
context creation fail with status -2 and a message, leave the CUDA error state
clean and the context usable; a BF16 Strassen product whose planes cannot be
allocated falls back to the classical kernel and counts a guard fall-back; and
`camblas_cuda_linear_bf16_static` makes no `cudaMalloc` call at all.
"""

import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_allocation_failures_are_reported_and_survivable(tmp_path):
    compiler = shutil.which("cc") or shutil.which("gcc")
    if not compiler:
        pytest.skip("needs a C compiler for the shim")
    shim = tmp_path / "alloc_fault_shim.so"
    subprocess.run([compiler, "-shared", "-fPIC", str(ROOT / "tests" / "alloc_fault_shim.c"), "-ldl",
                    "-o", str(shim)], check=True, capture_output=True, text=True)
    environment = dict(os.environ)
    environment["LD_PRELOAD"] = str(shim) + (":" + environment["LD_PRELOAD"]
                                             if environment.get("LD_PRELOAD") else "")
    done = subprocess.run([sys.executable, "-m", "tests.alloc_faults_child"], cwd=ROOT, env=environment,
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, (done.stdout + done.stderr)[-3000:]
    assert "alloc faults OK" in done.stdout
