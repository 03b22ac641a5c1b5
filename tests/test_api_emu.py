"""The library's C ABI called on a machine without a GPU (tests/api_emu.cu): every source of the
product library - the entry points of aotx_b200/csrc/q8_api.cu and q8_static.cu, the host
launch code, all kernels - compiled as host code around the stand-ins of tests/q8_ptx_emu.cuh,
with six emulated multiprocessors.  tests/test_stream_emu.py checks the kernels with arguments
its own driver fills in; here the library's host code fills them in, so these tests cover what
lies between the ABI and a launch: argument checks and return codes, the choice of kernel,
tensor maps (through a stand-in of the encoder that refuses what the driver refuses), grids,
scratch sets alternating between launches, workspaces, and
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
    done = subprocess.run([nvcc, "-O1", "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fno-strict-aliasing", "-gencode",
                           "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "aotx_b200", "csrc"),
                           "-I", os.path.join(ROOT, "tests"), "-o", path, os.path.join(ROOT, "tests", "api_emu.cu")],
                          capture_output=True, text=True, timeout=1200)
    assert done.returncode == 0, done.stderr[-3000:]
    lib = C.CDLL(path)
    library.declare_q8(lib)
    lib.api_emu_status.restype = C.c_uint
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


@pytest.mark.parametrize("m", [20, 50, 100])
def test_matmul_bfloat16_in_and_out(api, oracle, m):
    """20 rows: the x tiles are turned into binary16 in shared memory; 50 and 100 rows: x is
    turned once per launch into the context's binary16 copy before the product."""
    import aotx_b200
    import torch
    n, k = 300, 1024
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


@pytest.mark.parametrize("n,k,m", [(300, 1024, 20), (20, 96, 5)])
def test_fused_stores_on_both_kernel_families(api, n, k, m):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, 31)
    x = inputs(m, k, 32, scale=4.0)
    plain = np.zeros((m, n), np.float32)
    api.matmul(w, n, k, x, plain)
    y0 = np.random.default_rng(33).standard_normal((m + 1, n)).astype(np.float32)
    y = y0.copy()
    api.matmul(w, n, k, x, y, m=m, epilogue=1)
    assert np.array_equal(y[:m], y0[:m] + plain) and np.array_equal(y[m:], y0[m:])
    act = np.full((m + 1, n // 2), 9.0, np.float16)
    api.matmul(w, n, k, x, act, m=m, y_dtype=F16, epilogue=2)
    gate, up = plain[:, 0::2].astype(np.float64), plain[:, 1::2].astype(np.float64)
    want = gate / (1.0 + np.exp(-gate)) * up
    got = act[:m].astype(np.float64)
    assert (np.abs(got - want) <= 2.0 ** -10 * np.abs(want) + 1e-6).all()
    assert (act[m:] == np.float16(9.0)).all() and np.abs(want).max() > 0.1


def test_dequantisation_of_every_block_type(api, oracle):
    import aotx_b200
    from oracle.binding import row_bytes
    rows, k, first = 33, 512, 5
    w = aotx_b200.synth_q8_0(rows + first + 1, k, 70)
    out = np.full((rows + 1, k), 0x7777, np.uint16)
    assert api.lib.aotx_q8_dequant(api.ctx, None, w.ctypes.data, Q8_0, k, first, rows, out.ctypes.data) == OK
    api.clean()
    want = np.asarray(oracle.dequant(w, k, first, rows)).view(np.uint16).reshape(rows, k)
    assert np.array_equal(out[:rows], want) and (out[rows:] == 0x7777).all()
    rng = np.random.default_rng(71)
    for kind in sorted(_blocks.TYPES):
        n = 10
        blocks = _blocks.random_rows(kind, n, k, rng)
        out = np.full((7, k), 0x7777, np.uint16)
        assert api.lib.aotx_q8_dequant(api.ctx, None, blocks.ctypes.data, kind, k, 3, 6, out.ctypes.data) == OK
        api.clean()
        ideal = oracle.block_rows(kind, blocks, k, 3, 6)
        have = out[:6].view(np.float16).astype(np.float64)
        err = np.abs(have - ideal)
        assert ((err <= np.abs(ideal) * 9.765625e-04) | (err <= 5.9604644775390625e-08)).all(), kind
        assert (out[6:] == 0x7777).all()
        # and the product over that type
        x = inputs(9, k, 72 + kind)
        y = np.full((10, n), GUARD, np.float32)
        api.matmul(blocks, n, k, x, y, kind=kind, m=9)
        want = x.astype(np.float64) @ oracle.block_rows(kind, blocks, k, 0, n).T
        assert oracle.diff(y[:9], want)[0] == 0 and (y[9:] == GUARD).all(), kind
    assert api.lib.aotx_q8_dequant(api.ctx, None, w.ctypes.data, 9, k, 0, 1, out.ctypes.data) == ERR_TYPE


def moe_case(tokens, experts, used, hidden, ffn, seed):
    import aotx_b200
    wg = aotx_b200.synth_q8_0(experts * ffn, hidden, seed)
    wu = aotx_b200.synth_q8_0(experts * ffn, hidden, seed + 1)
    wd = aotx_b200.synth_q8_0(experts * hidden, ffn, seed + 2)
    rng = np.random.Generator(np.random.PCG64(seed + 3))
    x = rng.standard_normal((tokens, hidden)).astype(np.float16)
    router = (rng.standard_normal((experts, hidden)) / np.sqrt(hidden)).astype(np.float32)
    return wg, wu, wd, x, router


@pytest.mark.parametrize("tokens,experts,used,hidden,ffn", [(24, 5, 2, 256, 256), (5, 4, 2, 96, 64)])
def test_routed_expert_step_through_the_abi(api, oracle, tokens, experts, used, hidden, ffn):
    """Router, then the feed-forward step on the grouped tensor-core path (first shape) or on the
    per-pair kernels (second shape, which the grouped products do not take), the interleaved
    form, and the ordered sum alone."""
    import aotx_b200
    wg, wu, wd, x, router = moe_case(tokens, experts, used, hidden, ffn, 200 + tokens)
    prob = np.full((tokens + 1, experts), GUARD, np.float32)
    ids = np.full((tokens + 1, used), 0xFFFFFFFF, np.uint32)
    assert api.lib.aotx_q8_moe_route(api.ctx, None, x.ctypes.data, router.ctypes.data, tokens, None, hidden, experts,
                                     used, prob.ctypes.data, ids.ctypes.data) == OK
    api.clean()
    want_p, want_i = oracle.route(x.view(np.uint16), router, used)
    assert np.abs(prob[:tokens] - want_p).max() < 2e-6 and np.array_equal(ids[:tokens], want_i)
    assert (prob[tokens:] == GUARD).all() and (ids[tokens:] == 0xFFFFFFFF).all()
    prob, ids = np.ascontiguousarray(prob[:tokens]), np.ascontiguousarray(ids[:tokens])
    want = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x.view(np.uint16), prob, ids)
    space = api.workspace(tokens, used, hidden, ffn)

    def ffn_call(expect=OK, space=space, size=None):
        out = np.full((tokens + 1, hidden), GUARD, np.float32)
        code = api.lib.aotx_q8_moe_ffn(api.ctx, None, wg.ctypes.data, wu.ctypes.data, wd.ctypes.data, Q8_0, experts,
                                       hidden, ffn, x.ctypes.data, prob.ctypes.data, ids.ctypes.data, tokens, None,
                                       used, out.ctypes.data, F32, api.ptr(space),
                                       space.size if size is None else size)
        assert code == expect, code
        api.clean()
        return out

    out = ffn_call()
    ok, err, bound = oracle.within_bound(out[:tokens], want.astype(np.float64))
    assert ok, (err, bound)
    assert (out[tokens:] == GUARD).all()
    # workspace checks
    ffn_call(expect=ERR_WORKSPACE, size=space.size - 1)
    ffn_call(expect=ERR_WORKSPACE, space=None, size=0)
    if hidden % 256 == 0 and ffn % 256 == 0:
        both = aotx_b200.interleave_rows(wg, wu, hidden, groups=experts)
        out = np.full((tokens + 1, hidden), GUARD, np.float32)
        assert api.lib.aotx_q8_moe_ffn_fused(api.ctx, None, both.ctypes.data, wd.ctypes.data, Q8_0, experts, hidden,
                                             ffn, x.ctypes.data, prob.ctypes.data, ids.ctypes.data, tokens, None,
                                             used, out.ctypes.data, F32, space.ctypes.data, space.size) == OK
        api.clean()
        ok, err, bound = oracle.within_bound(out[:tokens], want.astype(np.float64))
        assert ok, (err, bound)
        assert (out[tokens:] == GUARD).all()
    else:
        both = np.zeros(16, np.uint8)
        out = np.zeros((tokens, hidden), np.float32)
        assert api.lib.aotx_q8_moe_ffn_fused(api.ctx, None, both.ctypes.data, wd.ctypes.data, Q8_0, experts, hidden,
                                             ffn, x.ctypes.data, prob.ctypes.data, ids.ctypes.data, tokens, None,
                                             used, out.ctypes.data, F32, space.ctypes.data,
                                             space.size) == ERR_UNSUPPORTED
    # the ordered sum alone, bit for bit
    rng = np.random.default_rng(5)
    proj = rng.standard_normal((tokens, used, hidden)).astype(np.float32)
    out = np.zeros((tokens, hidden), np.float32)
    assert api.lib.aotx_q8_moe_combine(api.ctx, None, proj.ctypes.data, prob.ctypes.data, ids.ctypes.data, tokens,
                                       None, hidden, experts, used, out.ctypes.data, F32) == OK
    api.clean()
    exact = oracle.ordered_sum(np.ascontiguousarray(proj.transpose(1, 0, 2)), prob, ids)
    assert np.array_equal(out.view(np.uint32), exact.view(np.uint32))


def test_entry_point_without_a_context(api, oracle):
    import aotx_b200
    n, k, m = 300, 1024, 20
    w = aotx_b200.synth_q8_0(n, k, 61)
    x = inputs(m, k, 62)
    want = oracle.product(w, n, k, x.view(np.uint16), m)
    for _ in range(2):
        y = np.full((m + 1, n), GUARD, np.float32)
        assert api.lib.aotx_q8_matmul_static(None, w.ctypes.data, Q8_0, n, k, x.ctypes.data, F16, m, None,
                                             y.ctypes.data, F32) == OK
        assert api.lib.api_emu_status() == 0
        assert oracle.diff(y[:m], want)[0] == 0 and (y[m:] == GUARD).all()
    big = inputs(65, k, 63)
    y = np.zeros((65, n), np.float32)
    assert api.lib.aotx_q8_matmul_static(None, w.ctypes.data, Q8_0, n, k, big.ctypes.data, F16, 65, None,
                                         y.ctypes.data, F32) != OK            # more rows than its scratch holds


def test_column_split_entry_point(api, oracle):
    import aotx_b200
    n, k, m, width, col0 = 300, 1024, 20, 900, 300
    w = aotx_b200.synth_q8_0(n, k, 71)
    x = inputs(m, k, 72)
    mine = np.full((m + 1, width), GUARD, np.float32)
    theirs = np.full((m + 1, width), GUARD, np.float32)
    table = (C.c_void_p * 2)(mine.ctypes.data, theirs.ctypes.data)
    assert api.lib.aotx_q8_matmul_peers(api.ctx, None, w.ctypes.data, Q8_0, n, k, x.ctypes.data, F16, m, None, table,
                                        2, width, col0, F32) == OK
    api.clean()
    want = oracle.product(w, n, k, x.view(np.uint16), m)
    for y in (mine, theirs):
        assert oracle.diff(y[:m, col0:col0 + n], want)[0] == 0
        assert (y[:m, :col0] == GUARD).all() and (y[:m, col0 + n:] == GUARD).all() and (y[m:] == GUARD).all()


def test_peer_barrier_passes_when_every_rank_arrived_and_gives_up_when_one_never_does(api):
    """aotx_q8_peer_barrier for rank 0 of two: it writes the step number into its word of both
    flag arrays; with rank 1's word already there it passes, and the step word counts up; with a
    rank that never arrives the bounded wait runs out, the flag-timeout bit is raised and the
    call still returns (the failure is made on the host: a word nothing writes)."""
    lib = api.lib
    lib.stream_emu_faults.argtypes = [C.c_longlong, C.c_double]
    mine = np.zeros(2, np.uint32)
    theirs = np.zeros(2, np.uint32)
    step = np.zeros(1, np.uint32)
    arrays = (C.c_void_p * 2)(mine.ctypes.data, theirs.ctypes.data)
    mine[1] = 1                                          # rank 1 has arrived for step 1
    assert lib.aotx_q8_peer_barrier(api.ctx, None, arrays, 2, 0, step.ctypes.data) == OK
    assert step[0] == 1 and mine[0] == 1 and theirs[0] == 1 and theirs[1] == 0
    status = C.c_uint32(9)
    assert lib.aotx_q8_device_status(api.ctx, C.byref(status), 1) == OK and status.value == 0
    # step 2: rank 1 never arrives
    lib.stream_emu_faults(-1, 0.3)
    try:
        assert lib.aotx_q8_peer_barrier(api.ctx, None, arrays, 2, 0, step.ctypes.data) == OK
    finally:
        lib.stream_emu_faults(-1, 10.0)
    assert step[0] == 2 and theirs[0] == 2
    assert lib.aotx_q8_device_status(api.ctx, C.byref(status), 1) != OK and status.value & 2
    assert lib.aotx_q8_device_status(api.ctx, C.byref(status), 1) == OK and status.value == 0
    # arguments
    assert lib.aotx_q8_peer_barrier(api.ctx, None, arrays, 2, 2, step.ctypes.data) == 1
    assert lib.aotx_q8_peer_barrier(api.ctx, None, arrays, 9, 0, step.ctypes.data) == 1
    assert lib.aotx_q8_peer_barrier(api.ctx, None, arrays, 2, 0, None) == 1
