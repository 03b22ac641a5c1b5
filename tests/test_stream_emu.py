"""The decode-regime tensor-core kernel run whole on the host (tests/stream_emu.cu): the source of
`q8_stream_kernel` (aotx_b200/csrc/q8_stream.cu) is compiled as host code, a block runs as its 480
host threads, and every instruction behind inline PTX is a host stand-in (tests/q8_ptx_emu.cuh) -
bulk tensor copies with the 128-byte swizzle, shared-memory barriers with arrival and byte counts,
tensor memory as an array, the MMA in float.  The results are checked against the oracle, so
this covers on a machine without a GPU what only the GPU tests covered before: the five warp
roles and their rings, the byte arithmetic of the dequantisation into tensor memory, the operand
layouts, the bfloat16 path, the unit schedule with tiles cut between blocks, the live batch word,
the three store modes.  In the asynchronous mode
the copies and the tensor-core work complete later, in order, on threads of their own with random
delays, so a buffer reused too early would give wrong numbers; and a copy that never lands (made
on the host) checks that every wait is bounded: the block raises its status bit, lets its other
copies land, hands its tensor memory back and ends.  The stand-ins also count uses that the
hardware does not define or faults on (tensor-memory lanes outside a warp's quarter, columns
outside the allocation, a bulk tensor copy whose inner coordinate is not a multiple of 16 bytes
or whose destination is off its boundary, an unaligned L2 request); any of them fails the launch
here (status 0x800).  The stand-ins encode what the instructions
do as the kernel was verified against the hardware; the hardware itself is the GPU tests'
matter."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GUARD = np.float32(-7.0)
ROWS, SEG_K, SEG_BYTES = 128, 256, 272


@pytest.fixture(scope="module")
def emu(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    path = str(tmp_path_factory.mktemp("emu") / "libstream_emu.so")
    done = subprocess.run([nvcc, "-O1", "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fno-strict-aliasing", "-gencode",
                           "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "aotx_b200", "csrc"),
                           "-I", os.path.join(ROOT, "tests"), "-o", path,
                           os.path.join(ROOT, "tests", "stream_emu.cu")],
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-3000:]
    lib = C.CDLL(path)
    vp, u32 = C.c_void_p, C.c_uint32
    lib.stream_emu.argtypes = [vp, u32, u32, vp, C.c_int, u32, vp, vp, u32, u32, u32, u32, C.c_int, u32]
    lib.stream_emu.restype = C.c_uint
    lib.stream_emu_faults.argtypes = [C.c_longlong, C.c_double]
    lib.stream_emu_form.argtypes = [C.c_uint]
    lib.stream_emu_copies.restype = C.c_longlong
    lib.stream_emu_peers.argtypes = [C.c_uint, vp, C.c_uint]
    lib.stream_emu_group_build.argtypes = [vp, u32, vp, u32, u32, u32, u32, u32, vp, vp, vp, vp]
    lib.stream_emu_moe.argtypes = [vp, vp, vp, vp, u32, u32, u32, vp, vp, u32, vp, u32, u32, u32, vp, vp, vp,
                                   C.c_int, u32]
    lib.stream_emu_moe.restype = C.c_uint
    lib.wide_emu.argtypes = [vp, u32, u32, vp, C.c_int, u32, vp, vp, u32, u32, C.c_int, u32]
    lib.wide_emu.restype = C.c_uint

    def run(w, n, k, x, y, bf16=0, live=None, mode=0, grid=5, ntok=16, delay_us=None, lost_copy=-1, expect=0,
            form=0):
        """delay_us: None runs copies and MMAs at once in the issuing thread, a number runs them
        later on engine threads with random delays up to that many microseconds."""
        m = x.shape[0]
        lib.stream_emu_faults(lost_copy, 10.0 if lost_copy < 0 else 0.5)
        lib.stream_emu_form(form)
        status = lib.stream_emu(w.ctypes.data, n, k, x.ctypes.data, bf16, m,
                                live.ctypes.data if live is not None else None, y.ctypes.data, y.shape[1], mode,
                                grid, ntok, 0 if delay_us is None else 1, delay_us or 0)
        lib.stream_emu_form(0)
        if expect is not None:
            assert status == expect, hex(status)
        return status

    def moe(wg, wu, both, wd, experts, hidden, ffn, x, ids, live=None, tile=64, grid=5, delay_us=None):
        """The routed-expert step; returns proj [tokens][used][hidden], act and the sorted pairs."""
        tokens, used = ids.shape
        proj = np.full((tokens * used, hidden), GUARD, np.float32)
        act = np.zeros((tokens * used, ffn), np.uint16)
        pair = np.full(tokens * used, 0xFFFFFFFF, np.uint32)
        ptr = lambda a: a.ctypes.data if a is not None else None
        lib.stream_emu_faults(-1, 10.0)
        status = lib.stream_emu_moe(ptr(wg), ptr(wu), ptr(both), ptr(wd), experts, hidden, ffn, x.ctypes.data,
                                    ids.ctypes.data, tokens, ptr(live), used, tile, grid, proj.ctypes.data,
                                    act.ctypes.data, pair.ctypes.data, 0 if delay_us is None else 1, delay_us or 0)
        run.copies = lib.stream_emu_copies()
        assert status == 0, hex(status)
        return proj.reshape(tokens, used, hidden), act, pair

    def wide(w, n, k, x, y, bf16=0, mode=0, grid=3, delay_us=None, live=None):
        """The prefill-regime kernel (token tiles of 256, weights in tensor memory)."""
        lib.stream_emu_faults(-1, 10.0)
        status = lib.wide_emu(w.ctypes.data, n, k, x.ctypes.data, bf16, x.shape[0],
                              live.ctypes.data if live is not None else None, y.ctypes.data, mode, grid,
                              0 if delay_us is None else 1, delay_us or 0)
        assert status == 0, hex(status)

    def peers(buffers, col0):
        """Column-split stores for the launches that follow: every tile goes to columns
        [col0, col0 + n) of each of the buffers; peers([], 0) switches it off."""
        table = (C.c_void_p * 8)(*[b.ctypes.data for b in buffers] + [None] * (8 - len(buffers)))
        lib.stream_emu_peers(len(buffers), table, col0)
    run.moe = moe
    run.wide = wide
    run.peers = peers
    run.lib = lib
    return run


def inputs(m, k, seed, scale=1.0):
    rng = np.random.Generator(np.random.PCG64(seed))
    return (rng.standard_normal((m, k)) * scale).astype(np.float16)


# shapes chosen so that tiles are cut between blocks, the last row tile is ragged, the batch does
# not fill its token tile, and (last three) there are several token tiles
SHAPES = [(200, 512, 5, 3, 16), (300, 1024, 20, 5, 32), (260, 768, 50, 4, 64), (130, 256, 100, 6, 128),
          (384, 2048, 33, 11, 16), (128, 256, 1, 1, 16), (1000, 512, 7, 9, 16), (300, 1024, 200, 7, 128),
          (140, 512, 70, 5, 32)]


@pytest.mark.parametrize("n,k,m,grid,ntok", SHAPES)
def test_product_against_the_oracle(emu, oracle, n, k, m, grid, ntok):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, n + k)
    x = inputs(m, k, m)
    y = np.full((m + 2, n), GUARD, np.float32)
    emu(w, n, k, x, y[:m], grid=grid, ntok=ntok)
    want = oracle.product(w, n, k, x.view(np.uint16), m)
    assert oracle.diff(y[:m], want)[0] == 0
    assert (y[m:] == GUARD).all()


@pytest.mark.parametrize("n,k,m,grid,ntok,delay", [(200, 512, 5, 3, 16, 0), (300, 1024, 20, 5, 32, 200),
                                                   (260, 768, 50, 4, 64, 100), (130, 256, 100, 6, 128, 100),
                                                   (384, 2048, 33, 11, 16, 50), (300, 1024, 200, 7, 128, 30)])
def test_copies_and_tensor_core_work_that_complete_later(emu, oracle, n, k, m, grid, ntok, delay):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, n + k)
    x = inputs(m, k, m)
    now = np.full((m, n), GUARD, np.float32)
    emu(w, n, k, x, now, grid=grid, ntok=ntok)
    later = np.full((m + 1, n), GUARD, np.float32)
    emu(w, n, k, x, later[:m], grid=grid, ntok=ntok, delay_us=delay)
    assert np.array_equal(later[:m], now)           # when an operation completes changes no bit
    assert (later[m:] == GUARD).all()
    assert oracle.diff(now, oracle.product(w, n, k, x.view(np.uint16), m))[0] == 0


@pytest.mark.parametrize("lost,delay", [(0, None), (1, 50), (7, None), (12, 50), (30, None)])
def test_a_copy_that_never_lands_ends_the_block_with_a_status(emu, lost, delay):
    """Copies alternate between the weight and the x thread, so the lost one is of either kind.
    Status bit 1: a barrier wait ran out; bit 2: the owner of a cut tile gave up on a partial sum
    (its holder had stopped); 0x100: a hand-over flag stayed raised, which the library's status
    call resets.  Never 0x200 (work in flight at the end) nor 0x400 (tensor memory kept)."""
    import aotx_b200
    n, k, m, grid, ntok = 300, 2048, 20, 5, 32
    w = aotx_b200.synth_q8_0(n, k, 5)
    x = inputs(m, k, 6)
    y = np.full((m + 1, n), GUARD, np.float32)
    status = emu(w, n, k, x, y[:m], grid=grid, ntok=ntok, delay_us=delay, lost_copy=lost, expect=None)
    assert status & 1
    assert status & ~0x103 == 0, hex(status)
    assert (y[m:] == GUARD).all()
    # the same launch without the fault is whole again
    good = np.zeros((m, n), np.float32)
    emu(w, n, k, x, good, grid=grid, ntok=ntok, delay_us=delay)


def test_one_block_and_many_blocks_agree_to_rounding(emu, oracle):
    import aotx_b200
    n, k, m = 300, 1536, 12
    w = aotx_b200.synth_q8_0(n, k, 3)
    x = inputs(m, k, 4)
    want = oracle.product(w, n, k, x.view(np.uint16), m)
    for grid in (1, 2, 7, 18):          # 18 = one block per unit
        y = np.zeros((m, n), np.float32)
        emu(w, n, k, x, y, grid=grid, ntok=16)
        assert oracle.diff(y, want)[0] == 0


@pytest.mark.parametrize("n,k,m,grid,ntok", [(200, 512, 9, 3, 16), (260, 768, 50, 4, 64), (130, 512, 100, 5, 128)])
def test_bfloat16_activations(emu, oracle, n, k, m, grid, ntok):
    import aotx_b200
    import torch
    w = aotx_b200.synth_q8_0(n, k, 11)
    xb = torch.from_numpy(inputs(m, k, 12).astype(np.float32)).to(torch.bfloat16)
    bits = np.ascontiguousarray(xb.view(torch.int16).numpy().view(np.uint16))
    y = np.full((m + 1, n), GUARD, np.float32)
    emu(w, n, k, bits, y[:m], bf16=1, grid=grid, ntok=ntok)
    # the kernel turns x into binary16 where it lies: exact for these magnitudes above 2^-14,
    # the few smaller ones round to the half subnormals
    x16 = xb.float().numpy().astype(np.float16)
    want = oracle.product(w, n, k, x16.view(np.uint16), m)
    assert oracle.diff(y[:m], want)[0] == 0
    assert (y[m:] == GUARD).all()


def test_live_batch_word(emu, oracle):
    import aotx_b200
    n, k, m = 200, 512, 40
    w = aotx_b200.synth_q8_0(n, k, 21)
    x = inputs(m, k, 22)
    full = np.zeros((m, n), np.float32)
    emu(w, n, k, x, full, grid=4, ntok=64)
    for live in (0, 1, 17, 40, 99):
        y = np.full((m, n), GUARD, np.float32)
        emu(w, n, k, x, y, live=np.array([live], np.uint32), grid=4, ntok=64)
        rows = min(live, m)
        # fewer live rows: the same sums (a row's sum does not depend on the other rows)
        assert np.array_equal(y[:rows], full[:rows])
        assert (y[rows:] == GUARD).all()


@pytest.mark.parametrize("n,k,m,grid,ntok", [(300, 1024, 20, 5, 32), (260, 768, 50, 4, 64), (200, 512, 5, 3, 16)])
def test_add_into_a_float_y(emu, n, k, m, grid, ntok):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, 31)
    x = inputs(m, k, 32)
    plain = np.zeros((m, n), np.float32)
    emu(w, n, k, x, plain, grid=grid, ntok=ntok)
    y0 = np.random.default_rng(33).standard_normal((m + 1, n)).astype(np.float32)
    y = y0.copy()
    emu(w, n, k, x, y[:m], mode=1, grid=grid, ntok=ntok)
    assert np.array_equal(y[:m], y0[:m] + plain)
    assert np.array_equal(y[m:], y0[m:])


@pytest.mark.parametrize("n,k,m,grid,ntok", [(300, 1024, 20, 5, 32), (256, 768, 50, 4, 64), (130, 512, 5, 3, 16)])
def test_gated_unit_over_row_pairs(emu, n, k, m, grid, ntok):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, 41)
    x = inputs(m, k, 42, scale=4.0)
    plain = np.zeros((m, n), np.float32)
    emu(w, n, k, x, plain, grid=grid, ntok=ntok)
    act = np.full((m + 1, n // 2), GUARD, np.float32)
    emu(w, n, k, x, act[:m], mode=2, grid=grid, ntok=ntok)
    gate, up = plain[:, 0::2].astype(np.float64), plain[:, 1::2].astype(np.float64)
    want = gate / (1.0 + np.exp(-gate)) * up
    assert np.abs(act[:m] - want).max() <= 2e-6 * np.abs(want).max()
    assert (act[m:] == GUARD).all()
    assert np.abs(want).max() > 0.1


def moe_case(oracle, tokens, experts, used, hidden, ffn, seed):
    import aotx_b200
    wg = aotx_b200.synth_q8_0(experts * ffn, hidden, seed)
    wu = aotx_b200.synth_q8_0(experts * ffn, hidden, seed + 1)
    wd = aotx_b200.synth_q8_0(experts * hidden, ffn, seed + 2)
    rng = np.random.Generator(np.random.PCG64(seed + 3))
    x = rng.standard_normal((tokens, hidden)).astype(np.float16)
    router = rng.standard_normal((experts, hidden)).astype(np.float32) / np.float32(np.sqrt(hidden))
    prob, ids = oracle.route(x.view(np.uint16), router, used)
    return wg, wu, wd, x, prob.astype(np.float32), ids


@pytest.mark.parametrize("tokens,experts,used,hidden,ffn,tile,grid", [(1, 5, 3, 512, 256, 64, 4),
                                                                      (33, 6, 2, 256, 256, 16, 5),
                                                                      (40, 3, 2, 512, 256, 32, 7),
                                                                      (90, 2, 1, 256, 512, 64, 3)])
def test_routed_experts_as_grouped_products(emu, oracle, tokens, experts, used, hidden, ffn, tile, grid):
    """Table build, row gather, the grouped mode of the tensor-core kernel over the table (with
    experts that got no token, token tiles that are not full and - last case - an expert with
    more than one token tile), the gated unit and the scatter through the row map; then the
    oracle's rank-ordered sum over the emulated projections against the oracle's whole step."""
    wg, wu, wd, x, prob, ids = moe_case(oracle, tokens, experts, used, hidden, ffn, 60 + tokens)
    proj, act, pair = emu.moe(wg, wu, None, wd, experts, hidden, ffn, x, ids, tile=tile, grid=grid)
    # a stable sort by expert: the place of a pair depends on the selections alone
    assert pair.tolist() == np.argsort(ids.reshape(-1), kind="stable").tolist()
    assert (proj != GUARD).all()
    again, _, _ = emu.moe(wg, wu, None, wd, experts, hidden, ffn, x, ids, tile=tile, grid=grid, delay_us=10)
    assert np.array_equal(again, proj)                     # run to run: the same bits
    got = oracle.ordered_sum(np.ascontiguousarray(proj.transpose(1, 0, 2)), prob, ids)
    want, want_act = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x.view(np.uint16), prob, ids, want_act=True)
    ok, err, bound = oracle.within_bound(got, want.astype(np.float64))
    assert ok, (err, bound)
    # the activations, pair by pair (the kernel keeps them in the sorted order)
    ours = act.view(np.float16).astype(np.float32)
    theirs = want_act.view(np.float16).astype(np.float32)           # [used][tokens][ffn]
    for at, p in enumerate(pair.tolist()):
        t, r = divmod(p, used)
        assert np.abs(ours[at] - theirs[r, t]).max() <= 2e-3 * np.abs(theirs[r, t]).max() + 1e-6


@pytest.mark.parametrize("tokens,experts,used,hidden,ffn,tile,grid,delay", [(33, 6, 2, 256, 256, 16, 5, None),
                                                                            (70, 3, 2, 512, 256, 64, 7, 50)])
def test_routed_experts_with_interleaved_gate_up(emu, oracle, tokens, experts, used, hidden, ffn, tile, grid, delay):
    import aotx_b200
    wg, wu, wd, x, prob, ids = moe_case(oracle, tokens, experts, used, hidden, ffn, 80 + tokens)
    both = aotx_b200.interleave_rows(wg, wu, hidden, groups=experts)
    plain, act0, pair0 = emu.moe(wg, wu, None, wd, experts, hidden, ffn, x, ids, tile=tile, grid=grid)
    fused, act1, pair1 = emu.moe(None, None, both, wd, experts, hidden, ffn, x, ids, tile=tile, grid=grid,
                                 delay_us=delay)
    order0, order1 = np.argsort(pair0), np.argsort(pair1)
    a0 = act0.view(np.float16).astype(np.float32)[order0]
    a1 = act1.view(np.float16).astype(np.float32)[order1]
    # the same sums cut at other points of the depth, then one rounding to half
    assert np.abs(a1 - a0).max() <= 2e-3 * np.abs(a0).max()
    assert np.abs(fused - plain).max() <= 1e-2 * np.abs(plain).max() + 1e-6
    got = oracle.ordered_sum(np.ascontiguousarray(fused.transpose(1, 0, 2)), prob, ids)
    want = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x.view(np.uint16), prob, ids)
    ok, err, bound = oracle.within_bound(got, want.astype(np.float64))
    assert ok, (err, bound)


def test_routed_experts_live_batch_and_selections_outside_the_table(emu, oracle):
    tokens, experts, used, hidden, ffn = 12, 4, 2, 256, 256
    wg, wu, wd, x, prob, ids = moe_case(oracle, tokens, experts, used, hidden, ffn, 99)
    whole, _, _ = emu.moe(wg, wu, None, wd, experts, hidden, ffn, x, ids, tile=16, grid=4)
    # fewer live tokens: their rows are the same, the others are not written
    part, _, _ = emu.moe(wg, wu, None, wd, experts, hidden, ffn, x, ids, live=np.array([5], np.uint32), tile=16,
                         grid=4)
    assert np.array_equal(part[:5], whole[:5]) and (part[5:] == GUARD).all()
    # a selection outside the expert table is left out; its projection row is never written
    bad = ids.copy()
    bad[3, 1] = experts + 7
    proj, _, pair = emu.moe(wg, wu, None, wd, experts, hidden, ffn, x, bad, tile=16, grid=4)
    assert (proj[3, 1] == GUARD).all()
    proj[3, 1] = whole[3, 1]
    assert np.array_equal(proj, whole)
    assert sorted(pair.tolist())[:-1] == [p for p in range(tokens * used) if p != 3 * used + 1]


@pytest.mark.parametrize("n,k,m,grid,delay", [(300, 1024, 300, 5, None), (520, 1024, 300, 3, 50),
                                              (390, 1024, 520, 4, 20), (128, 256, 257, 2, 0)])
def test_prefill_kernel_with_weights_in_tensor_memory(emu, oracle, n, k, m, grid, delay):
    """The prefill-regime kernel (aotx_b200/csrc/q8_wide.cu, batches above 128 rows):
    one accumulator, two segments of weights in tensor memory, x in boxes of 64 columns through a
    ring of its own, whole waves of tiles and a partial wave cut into units."""
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, 17)
    x = inputs(m, k, 18)
    y = np.full((m + 1, n), GUARD, np.float32)
    emu.wide(w, n, k, x, y[:m], grid=grid, delay_us=delay)
    assert oracle.diff(y[:m], oracle.product(w, n, k, x.view(np.uint16), m))[0] == 0
    assert (y[m:] == GUARD).all()
    # the live batch word and the add store
    live = m - 70
    part = np.full((m, n), GUARD, np.float32)
    emu.wide(w, n, k, x, part, grid=grid, delay_us=delay, live=np.array([live], np.uint32))
    assert (part[live:] == GUARD).all()
    if -(-live // 256) == -(-m // 256):
        assert np.array_equal(part[:live], y[:live])       # same tiles, same cuts, same sums
    else:
        assert np.abs(part[:live] - y[:live]).max() <= 1e-5 * np.abs(y[:m]).max()
    y0 = np.random.default_rng(19).standard_normal((m, n)).astype(np.float32)
    added = y0.copy()
    emu.wide(w, n, k, x, added, mode=1, grid=grid, delay_us=delay)
    assert np.array_equal(added, y0 + y[:m])


def test_prefill_kernel_with_weights_in_tensor_memory_bfloat16(emu, oracle):
    import aotx_b200
    import torch
    n, k, m = 260, 768, 270
    w = aotx_b200.synth_q8_0(n, k, 9)
    xb = torch.from_numpy(inputs(m, k, 10).astype(np.float32)).to(torch.bfloat16)
    bits = np.ascontiguousarray(xb.view(torch.int16).numpy().view(np.uint16))
    y = np.zeros((m, n), np.float32)
    emu.wide(w, n, k, bits, y, bf16=1, grid=4, delay_us=20)
    want = oracle.product(w, n, k, bits, m, bf16=True)
    assert oracle.diff(y, want)[0] == 0


# ---- the decode kernel for batches of up to 32 rows (aotx_b200/csrc/q8_decode.cu; form=1), on its
# ---- unit schedule (a cluster launch is not modelled by the emulation)

@pytest.mark.parametrize("n,k,m,grid,ntok,delay", [(200, 512, 5, 3, 16, None), (300, 1024, 20, 5, 32, 100),
                                                   (384, 2048, 12, 11, 16, 30), (128, 256, 1, 1, 16, None),
                                                   (1000, 512, 7, 9, 16, 0), (140, 512, 30, 5, 32, 20),
                                                   (300, 1536, 12, 18, 16, None)])
def test_decode_kernel_against_the_oracle(emu, oracle, n, k, m, grid, ntok, delay):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, n + k)
    x = inputs(m, k, m)
    runs = []
    for _ in range(2):
        y = np.full((m + 2, n), GUARD, np.float32)
        emu(w, n, k, x, y[:m], grid=grid, ntok=ntok, delay_us=delay, form=1)
        want = oracle.product(w, n, k, x.view(np.uint16), m)
        assert oracle.diff(y[:m], want)[0] == 0
        assert (y[m:] == GUARD).all()
        runs.append(y)
    # the sums run in a fixed order whatever the timing: the same bits every time
    assert np.array_equal(runs[0], runs[1])


def test_decode_kernel_bfloat16_live_batch_and_fused_stores(emu, oracle):
    import aotx_b200
    import torch
    n, k, m, grid, ntok = 300, 1024, 20, 5, 32
    w = aotx_b200.synth_q8_0(n, k, 31)
    xb = torch.from_numpy(inputs(m, k, 32).astype(np.float32)).to(torch.bfloat16)
    bits = np.ascontiguousarray(xb.view(torch.int16).numpy().view(np.uint16))
    y = np.full((m + 1, n), GUARD, np.float32)
    emu(w, n, k, bits, y[:m], bf16=1, grid=grid, ntok=ntok, form=1, delay_us=30)
    # binary16 weights; the bfloat16 x tile is turned into binary16 where it lies
    assert oracle.diff(y[:m], oracle.product(w, n, k, bits, m, bf16=True))[0] == 0
    assert (y[m:] == GUARD).all()
    x = inputs(m, k, 33, scale=4.0)
    plain = np.zeros((m, n), np.float32)
    emu(w, n, k, x, plain, grid=grid, ntok=ntok, form=1)
    for live in (0, 7, 20):
        part = np.full((m, n), GUARD, np.float32)
        emu(w, n, k, x, part, live=np.array([live], np.uint32), grid=grid, ntok=ntok, form=1)
        assert np.array_equal(part[:live], plain[:live]) and (part[live:] == GUARD).all()
    y0 = np.random.default_rng(34).standard_normal((m, n)).astype(np.float32)
    added = y0.copy()
    emu(w, n, k, x, added, mode=1, grid=grid, ntok=ntok, form=1)
    assert np.array_equal(added, y0 + plain)
    act = np.full((m + 1, n // 2), GUARD, np.float32)
    emu(w, n, k, x, act[:m], mode=2, grid=grid, ntok=ntok, form=1)
    gate, up = plain[:, 0::2].astype(np.float64), plain[:, 1::2].astype(np.float64)
    want = gate / (1.0 + np.exp(-gate)) * up
    assert np.abs(act[:m] - want).max() <= 2e-6 * np.abs(want).max()
    assert (act[m:] == GUARD).all()


@pytest.mark.parametrize("lost,delay", [(0, None), (3, 50), (11, None)])
def test_decode_kernel_a_copy_that_never_lands(emu, lost, delay):
    import aotx_b200
    n, k, m, grid, ntok = 300, 2048, 20, 5, 32
    w = aotx_b200.synth_q8_0(n, k, 5)
    x = inputs(m, k, 6)
    y = np.full((m + 1, n), GUARD, np.float32)
    status = emu(w, n, k, x, y[:m], grid=grid, ntok=ntok, delay_us=delay, lost_copy=lost, expect=None, form=1)
    assert status & 1
    assert status & ~0x103 == 0, hex(status)
    assert (y[m:] == GUARD).all()


@pytest.mark.parametrize("form", [0, 1])
def test_column_split_stores_into_every_peer(emu, oracle, form):
    """The store side of the column-split product: rank r computes columns [col0, col0 + n) and
    writes them into its own copy of the full y and into every peer's (ordinary stores through
    peer-mapped addresses on the GPU; here two host buffers).  Columns outside the slice and rows
    past the batch stay untouched in both."""
    import aotx_b200
    n, k, m, width, col0 = 300, 1024, 20, 900, 300
    w = aotx_b200.synth_q8_0(n, k, 61)
    x = inputs(m, k, 62)
    mine = np.full((m + 1, width), GUARD, np.float32)
    theirs = np.full((m + 1, width), GUARD, np.float32)
    unused = np.full((m, width), GUARD, np.float32)     # y itself is not written; its width is the row stride
    emu.peers([mine, theirs], col0)
    try:
        emu(w, n, k, x, unused, grid=5, ntok=32, form=form)
    finally:
        emu.peers([], 0)
    want = oracle.product(w, n, k, x.view(np.uint16), m)
    for y in (mine, theirs):
        assert oracle.diff(y[:m, col0:col0 + n], want)[0] == 0
        assert (y[:m, :col0] == GUARD).all() and (y[:m, col0 + n:] == GUARD).all() and (y[m:] == GUARD).all()
    assert np.array_equal(mine, theirs)
    assert (unused == GUARD).all()


@pytest.mark.parametrize("tokens,used,experts,tile", [(512, 8, 128, 64), (700, 3, 5, 16), (1, 8, 128, 64), (300, 4, 256, 32)])
def test_table_build_is_a_stable_sort_with_exact_tables(emu, tokens, used, experts, tile):
    """The table build on its own at sizes of several placement rounds (1024 pairs each): pairs
    sorted by expert in ascending pair order, selections outside the table left out, and the two
    tables equal to the ones written down here from the counts."""
    rng = np.random.default_rng(tokens + experts)
    ids = np.stack([rng.permutation(experts)[:used] for _ in range(tokens)]).astype(np.uint32)
    ids[rng.integers(tokens), rng.integers(used)] = experts + 1          # names no expert
    ffn, hidden = 768, 2048
    pairs = tokens * used
    pair = np.full(pairs, 0x55555555, np.uint32)
    room = (pairs // 16 + experts) * 16
    feed = np.zeros((room, 5), np.uint32)
    down = np.zeros((room, 5), np.uint32)
    counts = np.zeros(2, np.uint32)
    emu.lib.stream_emu_group_build(ids.ctypes.data, tokens, None, used, experts, ffn, hidden, tile, pair.ctypes.data,
                                   feed.ctypes.data, down.ctypes.data, counts.ctypes.data)
    flat = ids.reshape(-1)
    valid = np.nonzero(flat < experts)[0]
    order = valid[np.argsort(flat[valid], kind="stable")]
    assert pair[:len(order)].tolist() == order.tolist()
    assert (pair[len(order):] == 0xFFFFFFFF).all()
    want_feed, want_down, at = [], [], 0
    for e in range(experts):
        count = int((flat == e).sum())
        for tt in range(-(-count // tile)):
            tok0, limit = at + tt * tile, min(at + count, at + (tt + 1) * tile)
            want_feed += [(e * ffn + r * 128, r * 128, ffn, tok0, limit) for r in range(ffn // 128)]
            want_down += [(e * hidden + r * 128, r * 128, hidden, tok0, limit) for r in range(hidden // 128)]
        at += count
    assert counts.tolist() == [len(want_feed), len(want_down)]
    assert feed[:len(want_feed)].tolist() == [list(t) for t in want_feed]
    assert down[:len(want_down)].tolist() == [list(t) for t in want_down]


def test_benchmark_projection_at_full_size_and_grid(emu, oracle):
    """The O projection of the benchmark's decode step as it is launched: 4096 x 4096 weights, 32
    rows of binary16 x, 148 blocks (512 units, every block with a cut tile at both
    ends of its range), on both decode-regime kernels."""
    import aotx_b200
    n, k, m = 4096, 4096, 32
    w = aotx_b200.synth_q8_0(n, k, 77)
    x = inputs(m, k, 78)
    want = oracle.product(w, n, k, x.view(np.uint16), m)
    y = np.full((m + 1, n), GUARD, np.float32)
    emu(w, n, k, x, y[:m], grid=148, ntok=32)
    assert oracle.diff(y[:m], want)[0] == 0
    assert (y[m:] == GUARD).all()
    two = np.zeros((m, n), np.float32)
    emu(w, n, k, x, two, grid=296, ntok=32, form=1)
    assert oracle.diff(two, want)[0] == 0
