"""CPU-side checks: the library exports what the header declares, the layout helpers are
right, and the package refuses to run without a device (no fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from aotx_b200 import build
    return build.build()


def test_library_exports_every_declared_symbol(built):
    header = open(os.path.join(ROOT, "include", "aotx_q8_b200.h")).read()
    declared = set(re.findall(r"\b(aotx_q8_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 10
    lib = C.CDLL(built)
    for name in sorted(declared):
        assert hasattr(lib, name), name
    from aotx_b200.library import SYMBOLS
    assert declared == set(SYMBOLS)


def test_pack_unpack_round_trip_and_oracle_agreement(oracle):
    import aotx_b200
    rng = np.random.default_rng(1)
    n, k = 9, 128
    q = rng.integers(-127, 128, (n, k), dtype=np.int8)
    d = (rng.random((n, k // 32)) * 0.01).astype(np.float16)
    w = aotx_b200.pack_q8_0(q, d)
    assert w.size == n * aotx_b200.row_bytes(k) == n * 4 * 34
    q2, d2 = aotx_b200.unpack_q8_0(w, n, k)
    assert np.array_equal(q, q2) and np.array_equal(d.view(np.uint16), d2.view(np.uint16))
    want = (q.astype(np.float32).reshape(n, k // 32, 32) * d.astype(np.float32)[..., None])
    got = oracle.dequant(w, k, 0, n).view(np.float16)
    assert np.array_equal(got, want.astype(np.float16).reshape(n, k))


def test_synthetic_distribution():
    import aotx_b200
    w = aotx_b200.synth_q8_0(64, 1024, 0)
    q, d = aotx_b200.unpack_q8_0(w, 64, 1024)
    assert q.min() == -127 and q.max() == 127
    share = (d.astype(np.float32) < 6.1e-5).mean()
    assert 0.2 < share < 0.45
    assert np.array_equal(w, aotx_b200.synth_q8_0(64, 1024, 0))


def test_no_device_means_no_result():
    import torch
    import aotx_b200
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(RuntimeError):
        aotx_b200.Q8Context(0)


def test_product_package_never_touches_the_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, "aotx_b200")):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, name)).read()
                assert "oracle" not in text.replace("no CPU or PyTorch fallback", ""), name


def test_cpp_seam_compiles_and_links(built, tmp_path):
    """The C++ mirror of the reference's matrix seam builds against the header and links with
    the library (no device call is made)."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    src = tmp_path / "seam.cpp"
    src.write_text(
        '#include "aotx_b200_seam.hpp"\n'
        "int main(int argc, char **) {\n"
        "    aotx_b200_hold hold = {};\n"
        "    if (argc > 100) { aotx_model_matrix(&hold, 0, 8, 1, 32, 0, 1, 0, AOTX_B200_BATCH_TOKENS);\n"
        "        aotx_model_matrix_residual(&hold, 0, 8, 1, 32, 0, 1, 0, AOTX_B200_BATCH_TOKENS);\n"
        "        aotx_model_matrix_swiglu(&hold, 0, 8, 1, 32, 0, 1, 0, AOTX_B200_BATCH_TOKENS); }\n"
        "    return aotx_q8_set_path(0, 0) == AOTX_Q8_ERR_ARGUMENT ? 0 : 1;\n"
        "}\n")
    exe = tmp_path / "seam"
    cuda_inc = "/usr/local/cuda/include"
    lib_dir = os.path.dirname(built)
    subprocess.run(["g++", "-std=c++17", "-I" + os.path.join(ROOT, "include"), "-I" + cuda_inc, str(src),
                    "-o", str(exe), "-L" + lib_dir, "-laotx_q8_b200", "-Wl,-rpath," + lib_dir,
                    "-L/usr/local/cuda/lib64", "-lcudart"], check=True)
    assert subprocess.run([str(exe)]).returncode == 0


def test_cpp_seam_program_builds_and_fails_loudly_without_a_device(built, tmp_path):
    """The C++ parity program of the seam (run on the GPU by test_gpu_i_seam.py) compiles and
    links here; on a machine without a GPU its first call reports the CUDA error and stops."""
    import shutil
    import subprocess
    import torch
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    exe = tmp_path / "seam_check"
    lib_dir = os.path.dirname(built)
    subprocess.run([nvcc, "-O1", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
                    "-I", os.path.join(ROOT, "include"), "-o", str(exe),
                    os.path.join(ROOT, "tests", "seam_check.cu"), "-L", lib_dir, "-laotx_q8_b200",
                    "-Xlinker", "-rpath", "-Xlinker", lib_dir], check=True, timeout=900)
    if torch.cuda.is_available():
        return
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 1
    assert "aotx_q8_init" in run.stderr


def test_cpp_seam_program_dry_run(tmp_path):
    """The same program built with -DSEAM_DRY_RUN (tests/seam_dry.h: device memory is the heap,
    the captured graph is the recorded call replayed, the product is a host loop) runs to
    "pass": its fixtures, its host product, its measure, its guard rows and its loop over the
    batch word are sound.  The kernels are not involved."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    exe = tmp_path / "seam_dry"
    subprocess.run([nvcc, "-O2", "-std=c++17", "-DSEAM_DRY_RUN", "-diag-suppress", "550", "-gencode",
                    "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "include"),
                    "-I", os.path.join(ROOT, "tests"), "-o", str(exe),
                    os.path.join(ROOT, "tests", "seam_check.cu")], check=True, timeout=900)
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout[-2000:]
    lines = run.stdout.strip().splitlines()
    assert lines[-1] == "pass" and len(lines) == 11


def test_argument_checks_need_no_device(built):
    """Every entry point refuses bad arguments before it touches CUDA, so these calls are safe
    on a machine without a GPU: null context, wrong block type, depth not a multiple of 32, a
    batch beyond the fixed scratch of the context-free entry."""
    import aotx_b200
    lib = aotx_b200.load_library()
    null = C.c_void_p(None)
    one = C.c_void_p(256)  # never dereferenced: the checks below fail first
    assert lib.aotx_q8_set_path(null, 0) == 1
    assert lib.aotx_q8_set_overlap(null, 1) == 1
    assert lib.aotx_q8_dequant(null, null, one, 8, 64, 0, 1, one) == 1
    assert lib.aotx_q8_matmul(null, null, one, 8, 8, 64, one, 1, 1, None, one, 0) == 1
    assert lib.aotx_q8_moe_route(null, null, one, one, 1, None, 32, 4, 2, one, one) == 1
    assert lib.aotx_q8_moe_combine(null, null, one, one, one, 1, None, 32, 4, 2, one, 0) == 1
    assert lib.aotx_q8_matmul_static(null, one, 99, 8, 64, one, 1, 1, None, one, 0) == 2     # type
    assert lib.aotx_q8_matmul_static(null, one, 8, 8, 48, one, 1, 1, None, one, 0) == 1      # k % 32
    assert lib.aotx_q8_matmul_static(null, one, 8, 8, 64, one, 3, 1, None, one, 0) == 1      # x dtype
    assert lib.aotx_q8_matmul_static(null, one, 8, 8, 64, one, 1, 65, None, one, 0) == 5     # rows > 64
    assert lib.aotx_q8_matmul_static(null, one, 8, 0, 64, one, 1, 1, None, one, 0) == 0      # nothing to do
    assert lib.aotx_q8_matmul_fused(null, null, one, 8, 8, 64, one, 1, 1, None, one, 0, 1) == 1
    assert lib.aotx_q8_moe_ffn_fused(null, null, one, one, 8, 4, 256, 256, one, one, one, 1, None, 2, one, 0,
                                     one, 1 << 30) == 1
    small = lib.aotx_q8_moe_workspace_bytes(8, 2, 256, 256)
    large = lib.aotx_q8_moe_workspace_bytes(512, 8, 2048, 768)
    assert 0 < small < large and large % 256 == 0
    # the entries for several GPUs
    table = (C.c_void_p * 8)(*[C.c_void_p(256)] * 8)
    assert lib.aotx_q8_peer_barrier(null, null, table, 2, 0, one) == 1
    assert lib.aotx_q8_matmul_colsplit(null, null, one, 8, 8, 256, one, 1, 1, None, table, table, 2, 0, 16, 0, 0,
                                       one) == 1
    assert lib.aotx_q8_moe_ep(null, null, one, one, one, 8, 16, 512, 256, table, table, one, 4, 2, table, table, 2,
                              0, one, one, 0, one, 1 << 30) == 1
    assert lib.aotx_q8_moe_ep_workspace_bytes(4, 2, 512, 256, 0) == 0
    assert lib.aotx_q8_moe_ep_workspace_bytes(4, 2, 512, 256, 9) == 0
    two = lib.aotx_q8_moe_ep_workspace_bytes(64, 8, 2048, 768, 2)
    eight = lib.aotx_q8_moe_ep_workspace_bytes(64, 8, 2048, 768, 8)
    assert lib.aotx_q8_moe_workspace_bytes(128, 8, 2048, 768) < two < eight
    assert lib.aotx_q8_static_status(None, 0) != 0


def test_interleaved_rows_layout():
    """Row 2r of the interleaved tensor is gate row r, row 2r + 1 is up row r, expert by expert."""
    import aotx_b200
    k, ffn, experts = 64, 6, 3
    stride = aotx_b200.row_bytes(k)
    gate = aotx_b200.synth_q8_0(experts * ffn, k, 1)
    up = aotx_b200.synth_q8_0(experts * ffn, k, 2)
    both = aotx_b200.interleave_rows(gate, up, k, groups=experts).reshape(experts, ffn, 2, stride)
    assert np.array_equal(both[:, :, 0], gate.reshape(experts, ffn, stride))
    assert np.array_equal(both[:, :, 1], up.reshape(experts, ffn, stride))
    with pytest.raises(ValueError):
        aotx_b200.interleave_rows(gate, up[:stride], k)


def test_sharding_helpers_match_the_benchmark_shapes():
    from aotx_b200.sharded import ColumnSplit, shard_rows
    n, k = 151936, 8192
    total = 0
    for rank in range(8):
        b0, b1 = ColumnSplit.shard_bytes(n, k, 8, rank)
        assert b0 % 16 == 0 and (b1 - b0) == 18992 * (k // 32) * 34
        total += b1 - b0
    assert total == n * (k // 32) * 34
    assert shard_rows(128, 8, 7) == (112, 128)


def test_bench_accounting():
    """The byte and flop counts the benchmark divides by: every weight byte once plus
    activations in and results out; the fused layer reads and writes the float residual stream
    and writes one half per gate/up pair."""
    import importlib
    bench = importlib.import_module("bench")
    m, projections, _, _ = bench.WORKLOADS["decode_m32_llama3_8b_layer"]
    weights = sum(n * (k // 32) * 34 for _, k, n in projections)
    assert weights == 231735296                       # the four projections of the 8B layer
    plain = bench.algorithmic_bytes(m, projections, 2, 2)
    assert plain == weights + sum(m * k * 2 + m * n * 2 for _, k, n in projections)
    fused = bench.algorithmic_bytes(m, projections, 2, 2, fused=True)
    by_name = {name: (k, n) for name, k, n in projections}
    expect = weights + sum(m * k * 2 for _, k, _ in projections)
    expect += m * by_name["qkv"][1] * 2
    expect += 2 * m * by_name["o"][1] * 4 + 2 * m * by_name["down"][1] * 4
    expect += m * (by_name["gate_up"][1] // 2) * 2
    assert fused == expect
    assert bench.flops(m, projections) == sum(2 * m * n * k for _, k, n in projections)
    assert set(bench.FUSED) <= set(bench.WORKLOADS) and bench.TENSOR_BOUND <= set(bench.WORKLOADS)
