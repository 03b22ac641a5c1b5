"""The GPU tests that were written without a GPU at hand, run here against a CPU stand-in for
the device (tests/_fake.py, built on the oracle).  This checks the TESTS - argument names,
shapes, tolerances, guard rows, expected error codes - not the kernels; it keeps a test from
failing on its own mistakes the first time it meets a GPU."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(files, select=None):
    cmd = [sys.executable, "-m", "pytest", "--fake-device", "-m", "gpu", "-q", "-x", "-p", "no:cacheprovider"]
    if select:
        cmd += ["-k", select]
    cmd += [os.path.join(ROOT, "tests", name) for name in files]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, cwd=ROOT)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-1000:]
    return done.stdout


def test_upload_and_block_type_tests_are_sound():
    out = run(["test_gpu_g_gguf.py", "test_gpu_h_blocks.py"])
    assert " passed" in out and "failed" not in out


def test_fused_store_tests_are_sound():
    # the two long cases (the 8B gate+up shape, the 128-expert step) are left to the GPU
    out = run(["test_gpu_j_fused.py"], select="not 14336 and not 2048-768 and not 1024-512")
    assert " passed" in out and "failed" not in out
