"""The oracle restatement against the reference: golden fixtures (anywhere) and the
reference's own host functions compiled from its sources (where that library was built)."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle.binding import SEED, row_bytes


def test_random_generator_matches_golden(oracle, golden):
    state = C.c_uint64(SEED)
    draws = [oracle.lib.q8o_next(C.byref(state)) for _ in range(16)]
    assert np.array_equal(np.array(draws, np.uint64), golden["next_draws"])
    state = C.c_uint64(SEED)
    units = [oracle.lib.q8o_unit(C.byref(state)) for _ in range(16)]
    assert np.array_equal(np.array(units, np.float32), golden["unit_draws"])


def test_half_conversions_match_golden_and_numpy(oracle, golden):
    got = np.array([oracle.lib.q8o_f32_to_f16(float(v)) for v in golden["f2h_in"]], np.uint16)
    assert np.array_equal(got, golden["f2h_bits"])
    with np.errstate(over="ignore"):
        assert np.array_equal(got, golden["f2h_in"].astype(np.float16).view(np.uint16))
    back = np.array([oracle.lib.q8o_f16_to_f32(b) for b in range(65536)], np.float32)
    want = golden["h2f_all"]
    same = (back.view(np.uint32) == want.view(np.uint32)) | (np.isnan(back) & np.isnan(want))
    assert same.all()


def test_bf16_conversions_round_to_nearest_even(oracle):
    import torch
    rng = np.random.default_rng(3)
    vals = np.concatenate([rng.standard_normal(5000), rng.standard_normal(2000) * 1e-30,
                           rng.standard_normal(2000) * 1e30]).astype(np.float32)
    got = np.array([oracle.lib.q8o_f32_to_bf16(float(v)) for v in vals], np.uint16)
    want = torch.from_numpy(vals).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, want)
    back = np.array([oracle.lib.q8o_bf16_to_f32(int(b)) for b in got], np.float32)
    assert np.array_equal(back, torch.from_numpy(want.view(np.int16)).view(torch.bfloat16).float().numpy())


def test_fixture_builder_matches_golden(oracle, golden):
    assert np.array_equal(oracle.build(96, 256, SEED + 0), golden["dequant_w"])
    assert np.array_equal(oracle.build(80, 128, SEED + 8), golden["product_w"])
    assert np.array_equal(oracle.build(64, 64, SEED + 32), golden["turn_w"])
    assert np.array_equal(oracle.input(1, 128, SEED + 16), golden["product_x_m1"])
    assert np.array_equal(oracle.input(64, 128, SEED + 17), golden["product_x_m64"])
    assert np.array_equal(oracle.input(64, 64, SEED + 33), golden["turn_x"])


def test_dequant_bit_exact_with_golden(oracle, golden):
    w = golden["dequant_w"]
    for first, rows in ((16, 1), (16, 64), (0, 96)):
        got = oracle.dequant(w, 256, first, rows)
        assert np.array_equal(got, golden["dequant_want"][first:first + rows])


def test_dequant_matches_numpy_definition(oracle):
    rng = np.random.default_rng(11)
    n, k = 33, 512
    q = rng.integers(-127, 128, (n, k // 32, 32), dtype=np.int8)
    d = (np.abs(rng.normal(0, 0.02, (n, k // 32))) / 127).astype(np.float16)
    w = np.zeros((n, k // 32, 34), np.uint8)
    w[..., :2] = d.view(np.uint8).reshape(n, k // 32, 2)
    w[..., 2:] = q.view(np.uint8)
    want = (q.astype(np.float32) * d.astype(np.float32)[..., None]).astype(np.float16)
    got = oracle.dequant(w.reshape(-1), k, 0, n)
    assert np.array_equal(got, want.reshape(n, k).view(np.uint16))
    assert (d.astype(np.float32) < 6.1e-5).any(), "the distribution must reach half subnormals"


def test_product_bit_exact_with_golden(oracle, golden):
    for m in (1, 64):
        y = oracle.product(golden["product_w"], 80, 128, golden["product_x_m%d" % m], m)
        assert np.array_equal(y, golden["product_want_m%d" % m])
    y = oracle.product(golden["turn_w"], 64, 64, golden["turn_x"], 64)
    assert np.array_equal(y, golden["turn_want"])
    y = oracle.product(golden["turn_w"], 64, 64, golden["turn_x"], 64, swap=True)
    assert np.array_equal(y, golden["turn_want_swapped"])
    # the result must not depend on the thread split
    y1 = oracle.product(golden["turn_w"], 64, 64, golden["turn_x"], 64, threads=1)
    assert np.array_equal(y1, golden["turn_want"])


def test_turned_operand_is_detected(oracle, golden):
    """Negative arm of tests/matrix_test.cu:432-468."""
    got = golden["turn_want"].astype(np.float32)
    right, _ = oracle.diff(got, golden["turn_want"])
    turned, _ = oracle.diff(got, golden["turn_want_swapped"])
    assert right == 0 and turned > 0


def test_comparisons_match_golden(oracle, golden):
    got = (golden["turn_want"] * (1 + 3e-3)).astype(np.float32)
    bad, worst = oracle.diff(got, golden["turn_want"])
    assert [bad, worst] == list(golden["diff_probe"])
    bad, worst = oracle.spot(golden["turn_w"], 64, 64, golden["turn_x"], 64, got)
    assert [bad, worst] == list(golden["spot_probe"])
    nan = got.copy()
    nan.reshape(-1)[3] = np.nan
    bad, worst = oracle.diff(nan, golden["turn_want"])
    assert bad == 1 and np.isinf(worst)


def test_known_answer_vector(oracle):
    """tests/embedded_modules_test.cu:22-51: scale 1.0, row i all i+1, x all ones:
    y[i] = 32 * (i + 1)."""
    w = np.zeros((32, 34), np.uint8)
    w[:, 1] = 0x3C
    for i in range(32):
        w[i, 2:] = i + 1
    x = np.full((1, 32), 0x3C00, np.uint16)
    y = oracle.product(w.reshape(-1), 32, 32, x, 1)
    assert np.array_equal(y[0], 32.0 * np.arange(1, 33))


def test_against_reference_library(oracle, reference):
    """Direct comparison with the reference's compiled host functions on fresh seeds."""
    if not reference.available:
        pytest.skip("reference library not built on this machine")
    for n, k, seed in ((40, 256, SEED + 101), (7, 32, SEED + 5), (16, 1024, 12345)):
        w = reference.build(n, k, seed)
        assert np.array_equal(oracle.build(n, k, seed), w)
        x = reference.input(3, k, seed + 1)
        assert np.array_equal(oracle.input(3, k, seed + 1), x)
        want = reference.product(w, n, k, x, 3)
        assert np.array_equal(oracle.product(w, n, k, x, 3), want)
        deq = oracle.dequant(w, k, 0, n)
        assert reference.same(w, n, k, 0, n, deq) == 0
        got = (want * (1 - 2e-3)).astype(np.float32)
        assert oracle.diff(got, want) == reference.diff(got, want)
        assert oracle.spot(w, n, k, x, 3, got) == reference.spot(w, n, k, x, 3, got)
    rng = np.random.default_rng(5)
    for v in rng.standard_normal(3000).astype(np.float32) * np.float32(1e-4):
        assert oracle.lib.q8o_f32_to_f16(float(v)) == reference.lib.ref_float_to_half_bits(float(v))


def test_route_order_and_ties(oracle):
    """Fixture of tests/expert_test.cu:66-89: equal router rows 0 and 1 give a tie that the
    lower index wins; probabilities sum to one; selections are in falling probability."""
    for tokens, experts, used in ((1, 7, 1), (64, 7, 3), (64, 7, 7), (64, 64, 8), (5, 256, 256)):
        hidden = 32
        router = np.zeros((experts, hidden), np.float32)
        for e in range(experts):
            pos = np.float32(e) / np.float32(experts - 1)
            router[e] = [np.float32((d % 5) - 2) * np.float32(0.0012345) for d in range(hidden)]
            router[e, 0] = np.float32(3.0) * pos
            router[e, 1] = np.float32(-3.0) * pos * pos
        router[1] = router[0]
        x = np.zeros((tokens, hidden), np.float16)
        for t in range(tokens):
            x[t] = [(((t * 7 + d * 3) % 13) - 6) / 16.0 for d in range(hidden)]
            x[t, 0] = np.float32(2.0) * np.float32(t) / np.float32(tokens) + np.float32(0.007)
            x[t, 1] = 1.0
        prob, ids = oracle.route(x.view(np.uint16), router, used)
        assert np.allclose(prob.sum(1), 1.0, atol=1e-12)
        for t in range(tokens):
            order = sorted(range(experts), key=lambda e: (-prob[t, e], e))
            assert list(ids[t]) == order[:used]
            assert prob[t, 0] == prob[t, 1]
            if 1 in ids[t]:
                at = list(ids[t]).index(1)
                assert at > 0 and ids[t, at - 1] == 0
        assert np.array_equal(oracle.rank(prob.astype(np.float32), used)[:, :1], ids[:, :1]) or used > 1


def test_ordered_sum_is_rank_ordered_float(oracle):
    """tests/expert_test.cu:164-178: product and sum are rounded separately, rank by rank."""
    rng = np.random.default_rng(2)
    used, tokens, hidden, experts = 4, 3, 16, 6
    proj = rng.standard_normal((used, tokens, hidden)).astype(np.float32)
    prob = rng.random((tokens, experts)).astype(np.float32)
    ids = np.stack([rng.permutation(experts)[:used] for _ in range(tokens)]).astype(np.uint32)
    got = oracle.ordered_sum(proj, prob, ids)
    want = np.zeros((tokens, hidden), np.float32)
    for r in range(used):
        for t in range(tokens):
            p = (proj[r, t] * prob[t, ids[t, r]]).astype(np.float32)
            want[t] = p if r == 0 else (want[t] + p).astype(np.float32)
    assert np.array_equal(got, want)


def test_expert_matrix_slices(oracle):
    """tests/expert_test.cu:274-327 shape: 5 experts, used 3, n=19, k=512."""
    experts, used, n, k, tokens = 5, 3, 19, 512, 4
    w = oracle.build(experts * n, k, SEED + 77)
    x = oracle.input(tokens, k, SEED + 78)
    ids = np.array([[(t * 3 + r * 2 + 1) % experts for r in range(used)] for t in range(tokens)],
                   np.uint32)
    for rank in range(used):
        y, mag = oracle.expert_matrix(w, n, k, x, ids, rank)
        for t in range(tokens):
            e = int(ids[t, rank])
            slice_w = w[e * n * row_bytes(k):(e + 1) * n * row_bytes(k)]
            want = oracle.product(slice_w, n, k, x[t:t + 1], 1)
            # the slice check keeps the product un-rounded; the product reference rounds the
            # weight to half first: they agree to the half rounding
            assert np.all(np.abs(y[t] - want[0]) <= 6e-4 * mag[t] + 1e-12)


def test_routed_experts_against_reference_kernel_outputs(oracle):
    """The routed-expert half of the oracle against what the reference's own kernels produced on
    a GPU (tests/golden/reference_moe.npz, written by tests/golden/make_golden_moe.py from
    cuda/model/experts.cu, expert_matrix.cu and norm.cu compiled unmodified), with the
    reference's own tolerances (tests/expert_test.cu:131-150, 164-178, 309-319)."""
    import _moe_cases as cases
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_moe.npz")
    if not os.path.exists(path):
        pytest.skip("golden file not written yet")
    gold = dict(np.load(path))
    for tokens, experts, used, precision in cases.ROUTE_CASES:
        router, x = cases.route_fixture(tokens, experts, precision)
        tag = "route_%d_%d_%d_%d" % (tokens, experts, used, precision)
        prob, ids = oracle.route(x.view(np.uint16), router, used)
        assert np.array_equal(ids, gold[tag + "_ids"])
        assert np.abs(prob - gold[tag + "_prob"]).max() < 2e-6
        assert np.array_equal(oracle.rank(gold[tag + "_prob"], used), gold[tag + "_ids"])
        proj = cases.add_fixture(tokens, used)
        got = oracle.ordered_sum(proj, gold[tag + "_prob"], gold[tag + "_ids"])
        assert np.array_equal(got.view(np.uint32), gold[tag + "_sum"].view(np.uint32))
    c = cases.SLICE_CASE
    for tokens in (1, 64):
        w, x, ids = cases.slice_fixture(tokens)
        for rank in range(c["used"]):
            want, mag = oracle.expert_matrix(w, c["n"], c["k"], x.view(np.uint16), ids, rank)
            assert (np.abs(gold["slice_%d" % tokens][rank] - want) <= 2e-6 * mag + 2e-5).all()
    for name in cases.FFN_CASES:
        (tokens, experts, used, hidden, ffn), wg, wu, wd, x, router = cases.ffn_fixture(name)
        prob, ids = gold["ffn_%s_prob" % name], gold["ffn_%s_ids" % name]
        want_p, want_i = oracle.route(x.view(np.uint16), router, used)
        assert np.array_equal(ids, want_i)
        assert np.abs(prob - want_p).max() < 2e-6
        keep = np.arange(tokens) if name == "small" else gold["ffn_full_tokens"][:4]
        want = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, np.ascontiguousarray(x[keep]).view(np.uint16),
                              np.ascontiguousarray(prob[keep]), np.ascontiguousarray(ids[keep]))
        ref_sum = gold["ffn_small_sum"] if name == "small" else gold["ffn_full_sum"][:4]
        ok, err, bound = oracle.within_bound(ref_sum, want.astype(np.float64))
        assert ok, (name, err, bound)
        assert oracle.diff(ref_sum, want.astype(np.float64))[0] == 0
