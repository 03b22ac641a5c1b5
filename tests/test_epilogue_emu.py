"""The store side of the tensor-core kernels on the host (tests/epilogue_emu.cu): the source of
`epilogue_piece` (aotx_b200/csrc/q8_tile.cuh) runs as host threads, every block of a small grid
at once, with the hardware helpers it calls replaced by stand-ins, and each piece is handed
the accumulator its MMAs would have left.  Checked here: tiles cut between blocks are summed by
their owner and every output is stored exactly once, in the right row and column; rows past the
batch stay untouched; the row map of the grouped mode; the flags are handed back; and the
three store modes - plain, add into a float y (bit-identical with store-then-add), gated unit
over row pairs - for one and several token tiles and for 16, 32 and 64 columns per tile."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GUARD = np.float32(-12345.0)


@pytest.fixture(scope="module")
def emu(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    path = str(tmp_path_factory.mktemp("emu") / "libepilogue_emu.so")
    done = subprocess.run([nvcc, "-O1", "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fno-strict-aliasing", "-gencode",
                           "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "aotx_b200", "csrc"),
                           "-o", path, os.path.join(ROOT, "tests", "epilogue_emu.cu")],
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-3000:]
    lib = C.CDLL(path)
    vp, u32 = C.c_void_p, C.c_uint32
    lib.epilogue_emu.argtypes = [vp, u32, u32, vp, u32, vp, u32, u32, vp, u32, u32, u32]
    lib.epilogue_emu.restype = C.c_uint

    def run(w, x, y, mode=0, row_map=None, group=0, grid=5, ntok=32):
        n, k = w.shape
        m = x.shape[0]
        status = lib.epilogue_emu(w.ctypes.data, n, k, x.ctypes.data, m, y.ctypes.data, y.shape[1], mode,
                                  row_map.ctypes.data if row_map is not None else None, group, grid, ntok)
        assert status == 0, hex(status)
    return run


def case(n, k, m, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    return w, x, x.astype(np.float64) @ w.astype(np.float64).T


@pytest.mark.parametrize("n,k,m,grid,ntok", [(300, 1024, 20, 5, 32), (300, 1024, 70, 7, 32), (128, 512, 9, 3, 16),
                                             (260, 768, 50, 4, 64), (130, 256, 32, 6, 32), (300, 1024, 20, 1, 32),
                                             (384, 2048, 33, 11, 16)])
def test_plain_store(emu, n, k, m, grid, ntok):
    w, x, want = case(n, k, m, n + m)
    y = np.full((m + 2, n), GUARD, np.float32)
    emu(w, x, y[:m], grid=grid, ntok=ntok)
    assert np.abs(y[:m] - want).max() <= 1e-5 * np.abs(want).max()
    assert (y[m:] == GUARD).all()


@pytest.mark.parametrize("n,k,m,grid,ntok", [(300, 1024, 20, 5, 32), (260, 768, 50, 4, 64), (128, 512, 40, 3, 16)])
def test_add_into_a_float_y(emu, n, k, m, grid, ntok):
    w, x, _ = case(n, k, m, 3 * n + m)
    plain = np.zeros((m, n), np.float32)
    emu(w, x, plain, grid=grid, ntok=ntok)
    rng = np.random.default_rng(1)
    y0 = rng.standard_normal((m + 1, n)).astype(np.float32)
    y = y0.copy()
    emu(w, x, y[:m], mode=1, grid=grid, ntok=ntok)
    assert np.array_equal(y[:m], y0[:m] + plain)      # the same sums, one float add each
    assert np.array_equal(y[m:], y0[m:])


@pytest.mark.parametrize("n,k,m,grid,ntok", [(300, 1024, 20, 5, 32), (256, 768, 50, 4, 64), (130, 512, 40, 3, 16)])
def test_gated_unit_over_row_pairs(emu, n, k, m, grid, ntok):
    w, x, _ = case(n, k, m, 5 * n + m)
    x *= 4.0
    plain = np.zeros((m, n), np.float32)
    emu(w, x, plain, grid=grid, ntok=ntok)
    act = np.full((m + 1, n // 2), GUARD, np.float32)
    emu(w, x, act[:m], mode=2, grid=grid, ntok=ntok)
    gate, up = plain[:, 0::2], plain[:, 1::2]
    want = (gate / (np.float32(1.0) + np.exp(-gate))) * up
    assert np.abs(act[:m] - want).max() <= 1e-5 * np.abs(want).max()
    assert (act[m:] == GUARD).all() and np.abs(want).max() > 0.5


def test_grouped_mode_scatters_rows_through_the_map(emu):
    n, k, m = 300, 1024, 24
    w, x, want = case(n, k, m, 77)
    rng = np.random.default_rng(2)
    rows_y = 40
    row_map = rng.permutation(rows_y)[:m].astype(np.uint32)
    y = np.full((rows_y, n), GUARD, np.float32)
    emu(w, x, y, row_map=row_map, group=1, grid=5, ntok=32)
    assert np.abs(y[row_map] - want).max() <= 1e-5 * np.abs(want).max()
    untouched = np.setdiff1d(np.arange(rows_y), row_map)
    assert (y[untouched] == GUARD).all()
    # and with the gated unit, as the interleaved routed-expert step uses it
    act = np.full((rows_y, n // 2), GUARD, np.float32)
    emu(w, x, act, mode=2, row_map=None, group=1, grid=5, ntok=32)
    plain = np.zeros((m, n), np.float32)
    emu(w, x, plain, grid=5, ntok=32)
    gate, up = plain[:, 0::2], plain[:, 1::2]
    want_act = (gate / (np.float32(1.0) + np.exp(-gate))) * up
    assert np.abs(act[:m] - want_act).max() <= 1e-5 * max(np.abs(want_act).max(), 1e-3)
    assert (act[m:] == GUARD).all()
