"""The kernels that run on the ordinary cores, executed on the host by tests/simt_emu.cu (the
kernel source compiled as host code, a block as host threads, warp shuffles as barriers between
them) and checked against the oracle: the any-shape Q8_0 product, its two fused stores, the
dequantisation and product kernels of the other block types, the exact Q8_0 dequantisation
(bit for bit), the expert router, the per-pair expert products and the rank-ordered sum (bit for
bit, at both load widths).  This checks the kernels' index
arithmetic and data flow - which rows, which columns, which lane stores - on a machine without
a GPU; the GPU tests repeat the checks on the real thing."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

import _blocks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def emu(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    path = str(tmp_path_factory.mktemp("emu") / "libsimt_emu.so")
    done = subprocess.run([nvcc, "-O1", "-std=c++17", "-shared", "-Xcompiler", "-fPIC,-fno-strict-aliasing", "-gencode",
                           "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "aotx_b200", "csrc"),
                           "-I", os.path.join(ROOT, "tests"), "-o", path, os.path.join(ROOT, "tests", "simt_emu.cu")],
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stderr[-3000:]
    lib = C.CDLL(path)
    vp, u32 = C.c_void_p, C.c_uint32
    lib.emu_dequant_any.argtypes = [vp, u32, u32, u32, u32, vp, u32]
    lib.emu_gemv_any.argtypes = [vp, u32, u32, u32, vp, u32, vp, vp, u32, u32]
    lib.emu_gemv_any_bf16.argtypes = [vp, u32, u32, u32, vp, u32, vp, u32, u32]
    lib.emu_gemv_q8.argtypes = [vp, u32, u32, vp, u32, vp, vp, u32]
    lib.emu_gemv_q8_fused.argtypes = [vp, u32, u32, vp, u32, vp, vp, u32, u32]
    lib.emu_dequant_q8.argtypes = [vp, C.c_ulonglong, vp, C.c_int, u32]
    lib.emu_route.argtypes = [vp, vp, u32, vp, u32, u32, u32, vp, vp, u32]
    lib.emu_expert_pairs.argtypes = [vp, vp, vp, u32, u32, vp, vp, u32, u32, vp, u32, vp, vp, u32]
    lib.emu_expert_sum.argtypes = [vp, vp, vp, u32, vp, u32, u32, u32, vp, u32, u32]
    return lib


def inputs(m, k, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.standard_normal((m, k)).astype(np.float16)


@pytest.mark.parametrize("n,k,m,grid", [(20, 128, 3, 2), (9, 96, 11, 1), (17, 64, 8, 3)])
def test_q8_product_kernel(emu, oracle, n, k, m, grid):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, 5)
    x = inputs(m, k, 6)
    y = np.full((m + 1, n), -7.0, np.float32)
    emu.emu_gemv_q8(w.ctypes.data, n, k, x.ctypes.data, m, None, y.ctypes.data, grid)
    want = oracle.product(w, n, k, x.view(np.uint16), m)
    assert oracle.diff(y[:m], want)[0] == 0
    assert (y[m:] == -7.0).all()
    # the live batch word
    live = np.array([2], np.uint32)
    y2 = np.full((m, n), -7.0, np.float32)
    emu.emu_gemv_q8(w.ctypes.data, n, k, x.ctypes.data, m, live.ctypes.data, y2.ctypes.data, grid)
    assert np.array_equal(y2[:2], y[:2]) and (y2[2:] == -7.0).all()


@pytest.mark.parametrize("n,k,m,grid", [(20, 128, 3, 2), (12, 64, 10, 1)])
def test_q8_product_with_the_fused_stores(emu, oracle, n, k, m, grid):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, 7)
    x = (inputs(m, k, 8).astype(np.float32) * 8).astype(np.float16)
    plain = np.zeros((m, n), np.float32)
    emu.emu_gemv_q8(w.ctypes.data, n, k, x.ctypes.data, m, None, plain.ctypes.data, grid)
    # residual add: one float add of the same sum
    rng = np.random.default_rng(9)
    y0 = rng.standard_normal((m + 1, n)).astype(np.float32)
    y = y0.copy()
    emu.emu_gemv_q8_fused(w.ctypes.data, n, k, x.ctypes.data, m, None, y.ctypes.data, 1, grid)
    assert np.array_equal(y[:m], y0[:m] + plain) and np.array_equal(y[m:], y0[m:])
    # gated unit over row pairs: rows 2p, 2p + 1 -> column p
    act = np.full((m + 1, n // 2), 9.0, np.float16)
    emu.emu_gemv_q8_fused(w.ctypes.data, n, k, x.ctypes.data, m, None, act.ctypes.data, 2, grid)
    gate, up = plain[:, 0::2], plain[:, 1::2]
    want = (gate / (1.0 + np.exp(-gate)) * up).astype(np.float32)
    got = act[:m].astype(np.float32)
    assert (np.abs(got - want) <= 2.0 ** -10 * np.abs(want) + 1e-6).all()
    assert (act[m:] == np.float16(9.0)).all()
    assert np.abs(want).max() > 0.1


@pytest.mark.parametrize("kind", sorted(_blocks.TYPES))
def test_other_block_types_dequant_and_product(emu, oracle, kind):
    rng = np.random.default_rng(40 + kind)
    n, k, m = 10, 512, 9
    w = _blocks.random_rows(kind, n, k, rng)
    first, rows = 3, 6
    out = np.full((rows + 1, k), 0x7777, np.uint16)
    emu.emu_dequant_any(w.ctypes.data, kind, k, first, rows, out.ctypes.data, 2)
    ideal = oracle.block_rows(kind, w, k, first, rows)
    have = out[:rows].view(np.float16).astype(np.float64)
    err = np.abs(have - ideal)
    assert ((err <= np.abs(ideal) * 9.765625e-04) | (err <= 5.9604644775390625e-08)).all()
    assert (out[rows:] == 0x7777).all()
    x = inputs(m, k, 50 + kind)
    want = x.astype(np.float64) @ oracle.block_rows(kind, w, k, 0, n).T
    results = []
    for wide_x in (1, 0):      # 16-byte loads of x, and the element-wise path for an unaligned x
        y = np.full((m + 1, n), -7.0, np.float32)
        emu.emu_gemv_any(w.ctypes.data, kind, n, k, x.ctypes.data, m, None, y.ctypes.data, wide_x, 2)
        assert oracle.diff(y[:m], want)[0] == 0
        assert (y[m:] == -7.0).all()
        results.append(y)
    assert np.array_equal(results[0], results[1])
    # bfloat16 in and out
    import torch
    xb = torch.from_numpy(x.astype(np.float32)).to(torch.bfloat16)
    bits = xb.view(torch.int16).numpy().view(np.uint16)
    yb = np.zeros((m, n), np.uint16)
    emu.emu_gemv_any_bf16(w.ctypes.data, kind, n, k, bits.ctypes.data, m, yb.ctypes.data, 1, 2)
    got = torch.from_numpy(yb.view(np.int16)).view(torch.bfloat16).double().numpy()
    want_b = xb.double().numpy() @ oracle.block_rows(kind, w, k, 0, n).T
    assert np.abs(got - want_b).max() <= 1e-2 * np.abs(want_b).max() + 1e-3


@pytest.mark.parametrize("rows,k,first,wide", [(96, 256, 0, 1), (7, 64, 3, 0), (33, 4096, 5, 1)])
def test_q8_dequantisation_bit_for_bit(emu, oracle, rows, k, first, wide):
    """The byte-permute / half-subtract / half-multiply form of half(q * d) against the
    oracle's float product rounded once, subnormal scales and results included."""
    import aotx_b200
    from oracle.binding import row_bytes
    n = rows + first + 2
    w = aotx_b200.synth_q8_0(n, k, 70 + rows)
    out = np.full((rows + 1, k), 0x7777, np.uint16)
    base = w[first * row_bytes(k):]
    emu.emu_dequant_q8(base.ctypes.data, rows * (k // 32), out.ctypes.data, wide, 3)
    want = oracle.dequant(w, k, first, rows)
    assert np.array_equal(out[:rows], np.asarray(want).view(np.uint16).reshape(rows, k))
    assert (out[rows:] == 0x7777).all()


@pytest.mark.parametrize("tokens,experts,used,hidden", [(1, 7, 3, 32), (9, 64, 8, 96), (6, 256, 256, 64), (5, 3, 1, 32)])
def test_router(emu, oracle, tokens, experts, used, hidden):
    rng = np.random.default_rng(tokens + experts)
    x = rng.standard_normal((tokens, hidden)).astype(np.float16)
    router = (rng.standard_normal((experts, hidden)) / np.sqrt(hidden)).astype(np.float32)
    router[1] = router[0]                                  # a tie: the lower index ranks first
    prob = np.full((tokens + 1, experts), -7.0, np.float32)
    ids = np.full((tokens + 1, used), 0xFFFFFFFF, np.uint32)
    emu.emu_route(x.ctypes.data, router.ctypes.data, tokens, None, hidden, experts, used, prob.ctypes.data,
                  ids.ctypes.data, 2)
    want_p, want_i = oracle.route(x.view(np.uint16), router, used)
    assert np.abs(prob[:tokens] - want_p).max() < 2e-6
    assert np.array_equal(ids[:tokens], oracle.rank(prob[:tokens], used))
    assert np.array_equal(ids[:tokens], want_i)
    assert (prob[tokens:] == -7.0).all() and (ids[tokens:] == 0xFFFFFFFF).all()
    # the live batch word
    prob2 = np.full((tokens, experts), -7.0, np.float32)
    ids2 = np.full((tokens, used), 0xFFFFFFFF, np.uint32)
    live = np.array([tokens - 1], np.uint32)
    emu.emu_route(x.ctypes.data, router.ctypes.data, tokens, live.ctypes.data, hidden, experts, used,
                  prob2.ctypes.data, ids2.ctypes.data, 2)
    assert np.array_equal(prob2[:tokens - 1], prob[:tokens - 1]) and (prob2[tokens - 1:] == -7.0).all()


@pytest.mark.parametrize("hidden,width", [(96, 4), (96, 1), (34, 1), (2048, 4)])
def test_rank_ordered_sum_bit_for_bit(emu, oracle, hidden, width):
    rng = np.random.default_rng(hidden + width)
    tokens, experts, used = 9, 11, 5
    proj = rng.standard_normal((tokens, used, hidden)).astype(np.float32)
    prob = rng.random((tokens, experts)).astype(np.float32)
    ids = np.stack([rng.permutation(experts)[:used] for _ in range(tokens)]).astype(np.uint32)
    want = oracle.ordered_sum(np.ascontiguousarray(proj.transpose(1, 0, 2)), prob, ids)
    out = np.full((tokens + 1, hidden), -7.0, np.float32)
    emu.emu_expert_sum(proj.ctypes.data, prob.ctypes.data, ids.ctypes.data, tokens, None, hidden, experts, used,
                       out.ctypes.data, width, 4)
    assert np.array_equal(out[:tokens].view(np.uint32), want.view(np.uint32))
    assert (out[tokens:] == -7.0).all()
    # a selection outside the table adds nothing: the sum is that of the other ranks, in order
    bad = ids.copy()
    bad[2, 1] = experts + 3
    bad[4, 0] = 0xFFFFFFFF
    out2 = np.zeros((tokens, hidden), np.float32)
    emu.emu_expert_sum(proj.ctypes.data, prob.ctypes.data, bad.ctypes.data, tokens, None, hidden, experts, used,
                       out2.ctypes.data, width, 4)
    keep = [t for t in range(tokens) if t not in (2, 4)]
    assert np.array_equal(out2[keep], out[keep])
    for t, gone in ((2, 1), (4, 0)):
        ranks = [r for r in range(used) if r != gone]
        one = oracle.ordered_sum(np.ascontiguousarray(proj[t:t + 1, ranks].transpose(1, 0, 2)), prob[t:t + 1],
                                 np.ascontiguousarray(ids[t:t + 1, ranks]))
        assert np.array_equal(out2[t], one[0])          # 0 + v = v: the missing rank leaves no trace


def test_per_pair_expert_products(emu, oracle):
    import aotx_b200
    tokens, experts, used, hidden, ffn = 5, 4, 2, 64, 32
    wg = aotx_b200.synth_q8_0(experts * ffn, hidden, 1)
    wu = aotx_b200.synth_q8_0(experts * ffn, hidden, 2)
    wd = aotx_b200.synth_q8_0(experts * hidden, ffn, 3)
    rng = np.random.default_rng(4)
    x = rng.standard_normal((tokens, hidden)).astype(np.float16)
    router = (rng.standard_normal((experts, hidden)) / 8).astype(np.float32)
    prob, ids = oracle.route(x.view(np.uint16), router, used)
    prob = prob.astype(np.float32)
    act = np.zeros((tokens * used, ffn), np.uint16)
    proj = np.full((tokens * used + 1, hidden), -7.0, np.float32)
    emu.emu_expert_pairs(wg.ctypes.data, wu.ctypes.data, wd.ctypes.data, hidden, ffn, x.ctypes.data, ids.ctypes.data,
                         experts, tokens, None, used, act.ctypes.data, proj.ctypes.data, 3)
    assert (proj[tokens * used:] == -7.0).all()
    got = oracle.ordered_sum(np.ascontiguousarray(proj[:tokens * used].reshape(tokens, used, hidden).transpose(1, 0, 2)),
                             prob, ids)
    want = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x.view(np.uint16), prob, ids)
    ok, err, bound = oracle.within_bound(got, want.astype(np.float64))
    assert ok, (err, bound)
    # a selection outside the table: that pair's rows are never written, the others are the same
    bad = ids.copy()
    bad[1, 0] = experts
    proj2 = np.full((tokens * used, hidden), -7.0, np.float32)
    act2 = np.zeros_like(act)
    emu.emu_expert_pairs(wg.ctypes.data, wu.ctypes.data, wd.ctypes.data, hidden, ffn, x.ctypes.data, bad.ctypes.data,
                         experts, tokens, None, used, act2.ctypes.data, proj2.ctypes.data, 3)
    assert (proj2[1 * used + 0] == -7.0).all()
    proj2[1 * used + 0] = proj[1 * used + 0]
    assert np.array_equal(proj2, proj[:tokens * used])
