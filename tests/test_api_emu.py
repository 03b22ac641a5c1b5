"""The library's C ABI called on a machine without a GPU (tests/api_emu.cu): every source of the
product library - the entry points of aotx_b200/csrc/q8_api.cu and q8_static.cu, the host
launch code, all kernels - compiled as host code around the stand-ins of tests/q8_ptx_emu.cuh,
with six emulated multiprocessors.  tests/test_stream_emu.py checks the kernels with arguments
its own driver fills in; here the library's host code fills them in, so these tests cover what
lies between the ABI and a launch: argument checks and return codes, the choice of kernel,
tensor maps (through a stand-in of the encoder that refuses what the driver refuses), grids,
scratch sets alternating between launches, workspaces, the hint for the following product, and
the order of the launches of the routed-expert step.  Results are checked against the oracle."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

import _blocks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GUARD = np.float32(-7.0)
OK, ERR_ARGUMENT, ERR_TYPE, ERR_CUDA, ERR_UNSUPPORTED, ERR_WORKSPACE = 0, 1, 2, 3, 4, 5
F32, F16, BF16 = 0, 1, 2
Q8_0 = 8
NP_OF = {F32: np.float32, F16: np.float16}


class Emulated:
    """The entry points on numpy arrays; every call must leave the emulation's own status clean
    (no work in flight at a block's end, tensor memory returned, no undefined use)."""

    def __init__(self, lib):
        self.lib = lib
        self.ctx = C.c_void_p()
        assert lib.aotx_q8_init(C.byref(self.ctx), 0) == OK

    def close(self):
        assert self.lib.aotx_q8_destroy(self.ctx) == OK

    def clean(self):
        assert self.lib.api_emu_status() == 0
        status = C.c_uint32(99)
        assert self.lib.aotx_q8_device_status(self.ctx, C.byref(status), 1) == OK and status.value == 0

    @staticmethod
    def ptr(a):
        return a.ctypes.data if a is not None else None

    def matmul(self, w, n, k, x, y, x_dtype=F16, y_dtype=F32, live=None, kind=Q8_0, m=None, epilogue=None,
               expect=OK):
        m = x.shape[0] if m is None else m
        if epilogue is None:
            code = self.lib.aotx_q8_matmul(self.ctx, None, self.ptr(w), kind, n, k, self.ptr(x), x_dtype, m,
                                           self.ptr(live), self.ptr(y), y_dtype)
        else:
            code = self.lib.aotx_q8_matmul_fused(self.ctx, None, self.ptr(w), kind, n, k, self.ptr(x), x_dtype, m,
                                                 self.ptr(live), self.ptr(y), y_dtype, epilogue)
        assert code == expect, code
        self.clean()

    def workspace(self, tokens, used, hidden, ffn):
        size = self.lib.aotx_q8_moe_workspace_bytes(tokens, used, hidden, ffn)
        raw = np.zeros(size + 256, np.uint8)
        skip = (-raw.ctypes.data) % 256
        return raw[skip:skip + size]


@pytest.fixture(scope="module")
def api(tmp_path_factory):
    from aotx_b200 import library
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    path = str(tmp_path_factory.mktemp("emu") / "libapi_emu.so")
    done = subprocess.run([nvcc, "-O1", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-gencode",
                           "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "aotx_b200", "csrc"),
                           "-I", os.path.join(ROOT, "tests"), "-o", path, os.path.join(ROOT, "tests", "api_emu.cu")],
                          capture_output=True, text=True, timeout=1200)
    assert done.returncode == 0, done.stderr[-3000:]
    lib = C.CDLL(path)
    library.declare_q8(lib)
    lib.api_emu_status.restype = C.c_uint
    lib.api_emu_l2_bytes.restype = C.c_ulonglong
    lib.api_emu_mode.argtypes = [C.c_int, C.c_uint]
    for name in library.SYMBOLS:
        assert hasattr(lib, name), name
    emulated = Emulated(lib)
    yield emulated
    emulated.close()


def inputs(m, k, seed, scale=1.0):
    rng = np.random.Generator(np.random.PCG64(seed))
    return (rng.standard_normal((m, k)) * scale).astype(np.float16)


def bf16_bits(x16):
    import torch
    xb = torch.from_numpy(x16.astype(np.float32)).to(torch.bfloat16)
    return np.ascontiguousarray(xb.view(torch.int16).numpy().view(np.uint16)), xb


# tensor-core kernel at every token tile (k a multiple of 256), several token tiles of 128, and
# the any-shape kernel (k = 96; a weight pointer off the 16-byte boundary)
@pytest.mark.parametrize("n,k,m", [(300, 1024, 1), (300, 1024, 20), (260, 768, 50), (130, 512, 100), (200, 512, 300),
                                   (20, 96, 5)])
def test_matmul_against_the_oracle(api, oracle, n, k, m):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, n + k)
    x = inputs(m, k, m)
    want = oracle.product(w, n, k, x.view(np.uint16), m)
    y = np.full((m + 1, n), GUARD, np.float32)
    api.matmul(w, n, k, x, y, m=m)
    assert oracle.diff(y[:m], want)[0] == 0 and (y[m:] == GUARD).all()
    # half results, and a second and third launch (the scratch sets alternate)
    for _ in range(2):
        half = np.zeros((m, n), np.float16)
        api.matmul(w, n, k, x, half, y_dtype=F16)
        assert np.array_equal(half, y[:m].astype(np.float16))
    # the live batch word
    live = np.array([max(m - 3, 0)], np.uint32)
    part = np.full((m, n), GUARD, np.float32)
    api.matmul(w, n, k, x, part, live=live)
    rows = int(live[0])
    assert (part[rows:] == GUARD).all()
    if rows:
        assert np.abs(part[:rows] - y[:rows]).max() <= 1e-5 * np.abs(y[:m]).max()


def test_matmul_bfloat16_in_and_out(api, oracle):
    import aotx_b200
    import torch
    n, k, m = 300, 1024, 20
    w = aotx_b200.synth_q8_0(n, k, 3)
    bits, xb = bf16_bits(inputs(m, k, 4))
    y = np.zeros((m, n), np.uint16)
    api.matmul(w, n, k, bits, y, x_dtype=BF16, y_dtype=BF16)
    got = torch.from_numpy(y.view(np.int16)).view(torch.bfloat16).double().numpy()
    want = oracle.product(w, n, k, xb.float().numpy().astype(np.float16).view(np.uint16), m)
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max() + 1e-3


def test_return_codes_and_nothing_written(api):
    import aotx_b200
    n, k, m = 64, 256, 4
    w = aotx_b200.synth_q8_0(n, k, 1)
    x = inputs(m, k, 2)
    y = np.full((m, n), GUARD, np.float32)
    api.matmul(None, n, k, x, y, expect=ERR_ARGUMENT)
    api.matmul(w, n, k, None, y, m=m, expect=ERR_ARGUMENT)
    api.matmul(w, n, k, x, None, expect=ERR_ARGUMENT)
    api.matmul(w, n, 48, x, y, expect=ERR_ARGUMENT)                  # k not a multiple of 32
    api.matmul(w, n, k, x, y, x_dtype=F32, expect=ERR_ARGUMENT)
    api.matmul(w, n, k, x, y, y_dtype=7, expect=ERR_ARGUMENT)
    api.matmul(w, n, k, x, y, kind=9, expect=ERR_TYPE)              # no such block type
    api.matmul(w, n, k, x, y, epilogue=5, expect=ERR_ARGUMENT)
    api.matmul(w, n, k, x, np.zeros((m, n), np.float16), y_dtype=F16, epilogue=1, expect=ERR_ARGUMENT)
    api.matmul(w, 63, k, x, y, epilogue=2, expect=ERR_ARGUMENT)      # gated unit over an odd row count
    assert (y == GUARD).all()
    api.matmul(w, n, k, x, y, m=0)                                    # an empty batch is not an error
    assert (y == GUARD).all()
    # a forced kernel family that cannot take the shape
    assert api.lib.aotx_q8_set_path(api.ctx, 2) == OK
    try:
        w96 = aotx_b200.synth_q8_0(n, 96, 1)
        api.matmul(w96, n, 96, inputs(m, 96, 2), y, expect=ERR_UNSUPPORTED)
        assert (y == GUARD).all()
    finally:
        assert api.lib.aotx_q8_set_path(api.ctx, 0) == OK
    assert api.lib.aotx_q8_set_path(api.ctx, 9) == ERR_ARGUMENT
