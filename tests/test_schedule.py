"""The streaming kernel's division of work, checked on the host.

`schedule_check.cu` drives the kernel's own scheduling helpers (`unit_range`, `WorkIter`,
`last_holder` in aotx_b200/csrc/q8_tile.cuh) over a sweep of shapes and grid sizes and checks
that every unit is computed once, that a block publishes before it waits, that the owner
of a cut tile waits for exactly the blocks that hold the rest of it, and that the bytes a launch
asks L2 for on behalf of the next product are those of that product's first units.  The reference has no
counterpart: its product kernel launches one block for each tile of y (cuda/model/gemm.cu:2-3)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_division_of_work_on_the_host(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    exe = str(tmp_path / "schedule_check")
    build = subprocess.run(
        [nvcc, "-O2", "-std=c++17", "-diag-suppress", "20011", "-gencode", "arch=compute_100a,code=sm_100a",
         "-I", os.path.join(ROOT, "aotx_b200", "csrc"), "-o", exe,
         os.path.join(ROOT, "tests", "schedule_check.cu")],
        capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-2000:]
    assert run.stdout.startswith("ok ")
