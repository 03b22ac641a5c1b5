"""The routed-expert oracle and the product's routed-expert kernels against the reference's own
kernels (cuda/model/experts.cu:10-98, expert_matrix.cu:8-63, norm.cu:92-105, compiled unmodified
into oracle/_ref/libaotx_ref.so) run on the same device, and against the golden file written from
such a run (tests/golden/make_golden_moe.py).  Tolerances are the reference's own
(tests/expert_test.cu:131-150, 309-319): selections exact, probabilities within 2e-6, slice
products within 2e-6 * sum|product| + 2e-5, ordered sums bit for bit."""
import os

import numpy as np
import pytest

import _moe_cases as cases
from _util import dev, dev_weights, torch_mod

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_moe.npz")


@pytest.fixture(scope="module")
def ctx():
    import aotx_b200
    c = aotx_b200.Q8Context(0)
    yield c
    c.close()


@pytest.fixture(scope="module")
def experts_ref():
    from oracle.binding import ReferenceExperts
    try:
        return ReferenceExperts()
    except (RuntimeError, OSError) as why:
        pytest.skip("reference library not built: %s" % why)


@pytest.fixture(scope="module")
def golden_moe():
    if not os.path.exists(GOLDEN):
        pytest.skip("no golden file yet")
    return dict(np.load(GOLDEN))


@pytest.mark.parametrize("tokens,experts,used,precision", cases.ROUTE_CASES)
def test_route_and_ordered_sum(ctx, oracle, experts_ref, tokens, experts, used, precision):
    torch = torch_mod()
    router, x = cases.route_fixture(tokens, experts, precision)
    ref_p, ref_i = experts_ref.route(x, router, used, grid=tokens + 2 if tokens == 1 else 7)
    want_p, want_i = oracle.route(x.view(np.uint16), router, used)
    assert np.array_equal(ref_i, want_i)
    assert np.abs(ref_p - want_p).max() < 2e-6
    assert np.array_equal(oracle.rank(ref_p, used), ref_i)
    prob, ids = ctx.moe_route(dev(x), dev(router), used)
    torch.cuda.synchronize()
    got_p, got_i = prob.cpu().numpy(), ids.cpu().numpy().view(np.uint32)
    assert np.array_equal(got_i, ref_i)
    assert np.abs(got_p - ref_p).max() < 2e-6
    proj = cases.add_fixture(tokens, used)
    ref_sum = experts_ref.ordered_sum(proj, ref_p, ref_i)
    assert np.array_equal(oracle.ordered_sum(proj, ref_p, ref_i).view(np.uint32), ref_sum.view(np.uint32))
    out = ctx.moe_combine(dev(np.ascontiguousarray(proj.transpose(1, 0, 2))), dev(ref_p),
                          dev(ref_i.view(np.int32)))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), ref_sum.view(np.uint32))


@pytest.mark.parametrize("tokens", [1, 64])
def test_slice_product(oracle, experts_ref, tokens):
    w, x, ids = cases.slice_fixture(tokens)
    c = cases.SLICE_CASE
    for rank in range(c["used"]):
        got = experts_ref.expert_matrix(w, c["n"], c["k"], x, ids, rank, c["experts"])
        want, mag = oracle.expert_matrix(w, c["n"], c["k"], x.view(np.uint16), ids, rank)
        assert np.isfinite(got).all()
        assert (np.abs(got - want) <= 2e-6 * mag + 2e-5).all()


@pytest.mark.parametrize("name", ["small", "full"])
def test_whole_step(ctx, oracle, experts_ref, name):
    """The reference's route + per-rank loop, the oracle and the product's grouped path on one
    input: same selections; sums within the product bound of each other."""
    torch = torch_mod()
    (tokens, experts, used, hidden, ffn), wg, wu, wd, x, router = cases.ffn_fixture(name)
    ref = experts_ref.ffn(wg, wu, wd, experts, hidden, ffn, x, router, used)
    keep = np.arange(tokens) if name == "small" else cases.full_sample_tokens(tokens)
    want = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, np.ascontiguousarray(x[keep]).view(np.uint16),
                          np.ascontiguousarray(ref["prob"][keep]), np.ascontiguousarray(ref["ids"][keep]))
    ok, err, bound = oracle.within_bound(ref["sum"][keep], want.astype(np.float64))
    assert ok, (err, bound)
    assert oracle.diff(ref["sum"][keep], want.astype(np.float64))[0] == 0
    xd = dev(x)
    prob, ids = ctx.moe_route(xd, dev(router), used)
    out = ctx.moe_ffn(dev_weights(wg), dev_weights(wu), dev_weights(wd), experts, hidden, ffn, xd, prob, ids)
    torch.cuda.synchronize()
    assert np.array_equal(ids.cpu().numpy().view(np.uint32), ref["ids"])
    got = out.cpu().numpy()
    ok, err, bound = oracle.within_bound(got, ref["sum"].astype(np.float64))
    assert ok, (err, bound)
    ok, err, bound = oracle.within_bound(got[keep], want.astype(np.float64))
    assert ok, (err, bound)
    assert oracle.diff(got[keep], want.astype(np.float64))[0] == 0
    assert ctx.device_status() == 0


def test_golden_file_matches_this_device(experts_ref, golden_moe):
    """The committed vectors are what the reference's kernels give here too (bit for bit: same
    kernels, same inputs, same order of sums)."""
    for tokens, experts, used, precision in cases.ROUTE_CASES:
        router, x = cases.route_fixture(tokens, experts, precision)
        prob, ids = experts_ref.route(x, router, used, grid=tokens + 2 if tokens == 1 else 7)
        tag = "route_%d_%d_%d_%d" % (tokens, experts, used, precision)
        assert np.array_equal(golden_moe[tag + "_ids"], ids)
        assert np.array_equal(golden_moe[tag + "_prob"].view(np.uint32), prob.view(np.uint32))


def test_single_row_module(oracle, reference):
    """The reference's PTX module (ptx/gemv_q8.ptx:18-223), assembled for this device, on its own
    known-answer shape and on a seeded 4096 x 4096 tensor: within the reference's measure of the
    oracle's product, and the product kernel agrees with it."""
    import aotx_b200
    import ctypes as C
    from oracle import build
    torch = torch_mod()
    if not getattr(reference, "available", False) or not os.path.exists(build.REF_MODULE):
        pytest.skip("reference module not built")
    lib = reference.lib
    lib.ref_gpu_module_open.restype = C.c_int
    lib.ref_gpu_module_open.argtypes = [C.c_char_p]
    lib.ref_gpu_module_gemv.restype = C.c_int
    lib.ref_gpu_module_gemv.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p]
    torch.zeros(1, device="cuda")
    assert lib.ref_gpu_module_open(build.REF_MODULE.encode()) == 0
    n = k = 4096
    w = aotx_b200.synth_q8_0(n, k, 5)
    x = np.random.Generator(np.random.PCG64(6)).standard_normal((1, k)).astype(np.float16)
    wd, xd = dev_weights(w), dev(x)
    y = torch.zeros(1, n, dtype=torch.float32, device="cuda")
    one = torch.ones(1, dtype=torch.int32, device="cuda")
    assert lib.ref_gpu_module_gemv(wd.data_ptr(), n, k, xd.data_ptr(), y.data_ptr(), one.data_ptr(), None) == 0
    torch.cuda.synchronize()
    want = oracle.product(w, n, k, x.view(np.uint16), 1)
    assert oracle.diff(y.cpu().numpy(), want)[0] == 0
    ctx = aotx_b200.Q8Context(0)
    ours = ctx.matmul(wd, n, k, xd, y=torch.zeros(1, n, dtype=torch.float32, device="cuda"))
    torch.cuda.synchronize()
    assert oracle.diff(ours.cpu().numpy(), want)[0] == 0
    ctx.close()
