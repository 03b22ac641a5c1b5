"""The C++ mirror of the reference's matrix seam, run on the GPU from a C++ program.

`seam_check.cu` calls `aotx_model_matrix` (include/aotx_b200_seam.hpp; reference
cuda/model/graph_host.h:47-52) the two ways the reference does: directly on a stream with a
host batch, as tests/matrix_test.cu drives the kernels, and inside an open stream capture
with the batch in a device word that changes between replays of the one graph
(cuda/model/graph_host.cu:20-40).  It checks every case against a host product in double with
the reference's measure and checks that rows past the batch keep their guard value."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_seam_from_cpp(tmp_path):
    import aotx_b200.library as library
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    lib_dir = os.path.dirname(library.LIB_PATH)
    assert os.path.exists(library.LIB_PATH)
    exe = str(tmp_path / "seam_check")
    build = subprocess.run(
        [nvcc, "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
         "-I", os.path.join(ROOT, "include"), "-o", exe, os.path.join(ROOT, "tests", "seam_check.cu"),
         "-L", lib_dir, "-laotx_q8_b200", "-Xlinker", "-rpath", "-Xlinker", lib_dir],
        capture_output=True, text=True, timeout=900)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, (run.stdout[-3000:], run.stderr[-2000:])
    assert run.stdout.strip().endswith("pass")
