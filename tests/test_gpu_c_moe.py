"""Routed experts on the device against the oracle (cases of tests/expert_test.cu)."""
import numpy as np
import pytest

from _util import GUARD, dev, dev_weights, torch_mod
from oracle.binding import SEED, row_bytes

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import aotx_b200
    c = aotx_b200.Q8Context(0)
    yield c
    c.close()


def _route_fixture(tokens, experts, precision):
    """Router rows and inputs of tests/expert_test.cu:66-89."""
    hidden = 32
    router = np.zeros((experts, hidden), np.float32)
    for e in range(experts):
        pos = np.float32(e) / np.float32(max(experts - 1, 1))
        for d in range(hidden):
            router[e, d] = (np.float32(1.0002) if e == 2 else np.float32(1.0)) if precision \
                else np.float32((d % 5) - 2) * np.float32(0.0012345)
        if not precision:
            router[e, 0] = np.float32(3.0) * pos
            router[e, 1] = np.float32(-3.0) * pos * pos
    router[1] = router[0]
    x = np.zeros((tokens, hidden), np.float16)
    for t in range(tokens):
        for d in range(hidden):
            x[t, d] = 1.0 if precision else (((t * 7 + d * 3) % 13) - 6) / 16.0
        if not precision:
            x[t, 0] = np.float32(2.0) * np.float32(t) / np.float32(tokens) + np.float32(0.007)
            x[t, 1] = 1.0
    return router, x


@pytest.mark.parametrize("tokens", [1, 64])
@pytest.mark.parametrize("experts,used,precision", [(7, 1, 0), (7, 3, 0), (7, 7, 0), (64, 8, 0),
                                                    (256, 256, 0), (3, 1, 1)])
def test_route(ctx, oracle, tokens, experts, used, precision):
    torch = torch_mod()
    router, x = _route_fixture(tokens, experts, precision)
    cap = tokens + 2
    prob = torch.full((cap, experts), GUARD, dtype=torch.float32, device="cuda")
    ids = torch.full((cap, used), -1, dtype=torch.int32, device="cuda")
    xd = dev(np.concatenate([x, np.zeros((2, 32), np.float16)]))
    ctx.moe_route(xd, dev(router), used, tokens=tokens, prob=prob, ids=ids)
    torch.cuda.synchronize()
    got_p = prob.cpu().numpy()
    got_i = ids.cpu().numpy().view(np.uint32)
    want_p, want_i = oracle.route(x.view(np.uint16), router, used)
    assert np.isfinite(got_p[:tokens]).all()
    assert np.abs(got_p[:tokens] - want_p).max() < 2e-6
    assert np.array_equal(got_i[:tokens], want_i)
    assert np.array_equal(got_i[:tokens], oracle.rank(got_p[:tokens], used))
    assert (got_p[tokens:] == GUARD).all() and (got_i[tokens:] == 0xFFFFFFFF).all()
    mass = np.take_along_axis(got_p[:tokens], got_i[:tokens].astype(np.int64), 1).sum(1)
    if used == experts:
        assert np.abs(mass - 1.0).max() < 2e-5
    else:
        assert (mass < 0.999).all()


def _moe_case(oracle, tokens, experts, used, hidden, ffn, seed):
    import aotx_b200
    wg = aotx_b200.synth_q8_0(experts * ffn, hidden, seed)
    wu = aotx_b200.synth_q8_0(experts * ffn, hidden, seed + 1)
    wd = aotx_b200.synth_q8_0(experts * hidden, ffn, seed + 2)
    rng = np.random.Generator(np.random.PCG64(seed + 3))
    # scales of the benchmark's distribution give outputs near 1e-4; a unit-size input keeps
    # every intermediate inside the half range
    x = rng.standard_normal((tokens, hidden)).astype(np.float16)
    router = rng.standard_normal((experts, hidden)).astype(np.float32) / np.float32(np.sqrt(hidden))
    return wg, wu, wd, x, router


@pytest.mark.parametrize("tokens,experts,used,hidden,ffn", [(1, 5, 3, 512, 64), (64, 5, 3, 512, 96),
                                                            (33, 16, 4, 256, 256), (200, 7, 2, 512, 256),
                                                            (64, 128, 8, 2048, 768)])
def test_moe_ffn_matches_oracle(ctx, oracle, tokens, experts, used, hidden, ffn):
    torch = torch_mod()
    wg, wu, wd, x, router = _moe_case(oracle, tokens, experts, used, hidden, ffn, 40 + tokens)
    xd = dev(x)
    prob, ids = ctx.moe_route(xd, dev(router), used)
    out = torch.full((tokens + 2, hidden), GUARD, dtype=torch.float32, device="cuda")
    ctx.moe_ffn(dev_weights(wg), dev_weights(wu), dev_weights(wd), experts, hidden, ffn, xd, prob,
                ids, tokens=tokens, out=out[:tokens])
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    p = prob.cpu().numpy()
    i = ids.cpu().numpy().view(np.uint32)
    want = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x.view(np.uint16), p, i)
    ok, err, bound = oracle.within_bound(got[:tokens], want.astype(np.float64))
    assert ok, (err, bound)
    assert oracle.diff(got[:tokens], want.astype(np.float64))[0] == 0
    assert (got[tokens:] == GUARD).all()


def test_selection_outside_the_expert_table_adds_nothing(ctx, oracle):
    """The selections come from the caller: one that names no expert is left out of the products
    (no kernel indexes a tensor with it) and adds nothing to its token's sum, on the grouped
    tensor-core path and on the per-pair path.  The reference has no such case: its selections
    come from its own router (cuda/model/experts.cu:10-75)."""
    import aotx_b200
    torch = torch_mod()
    tokens, experts, used, hidden, ffn = 24, 6, 2, 256, 256
    wg, wu, wd, x, router = _moe_case(oracle, tokens, experts, used, hidden, ffn, 77)
    xd = dev(x)
    prob, ids = ctx.moe_route(xd, dev(router), used)
    p = prob.cpu().numpy()
    i = ids.cpu().numpy().view(np.uint32)
    want = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x.view(np.uint16), p, i)
    first = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x.view(np.uint16), p, np.ascontiguousarray(i[:, :1]))
    want[3] = first[3]
    bad = i.copy()
    bad[3, 1] = 0xFFFFFFFF
    bad_dev = dev(bad.view(np.int32))
    dwg, dwu, dwd = dev_weights(wg), dev_weights(wu), dev_weights(wd)
    for path in (0, aotx_b200.PATH_GENERAL):
        ctx.set_path(path)
        try:
            out = ctx.moe_ffn(dwg, dwu, dwd, experts, hidden, ffn, xd, prob, bad_dev)
        finally:
            ctx.set_path(0)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        ok, err, bound = oracle.within_bound(got, want.astype(np.float64))
        assert ok, (path, err, bound)
    assert ctx.device_status() == 0


def test_ordered_sum_bit_exact(ctx, oracle):
    """The rank-ordered weighted sum equals the oracle bit for bit, rows past the batch stay
    untouched (tests/expert_test.cu:164-195)."""
    torch = torch_mod()
    rng = np.random.Generator(np.random.PCG64(3))
    for tokens, hidden, experts, used in ((1, 32, 7, 1), (9, 96, 11, 5), (64, 32, 7, 7)):
        proj = rng.standard_normal((tokens, used, hidden)).astype(np.float32)
        prob = rng.random((tokens, experts)).astype(np.float32)
        ids = np.stack([rng.permutation(experts)[:used] for _ in range(tokens)]).astype(np.uint32)
        want = oracle.ordered_sum(np.ascontiguousarray(proj.transpose(1, 0, 2)), prob, ids)
        out = torch.full((tokens + 2, hidden), GUARD, dtype=torch.float32, device="cuda")
        ctx.moe_combine(dev(proj), dev(prob), dev(ids.view(np.int32)), out=out[:tokens])
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert np.array_equal(got[:tokens].view(np.uint32), want.view(np.uint32))
        assert (got[tokens:] == GUARD).all()


def test_grouped_path_equals_per_pair_path_at_full_size(ctx, oracle):
    """The benchmark's routed-expert shape (512 tokens, 128 experts, top 8, 2048 -> 768 -> 2048):
    the grouped tensor-core path and the per-pair path give the same result within the product
    bound, and the same selections feed both."""
    import aotx_b200
    torch = torch_mod()
    tokens, experts, used, hidden, ffn = 512, 128, 8, 2048, 768
    wg, wu, wd, x, router = _moe_case(oracle, tokens, experts, used, hidden, ffn, 900)
    xd = dev(x)
    prob, ids = ctx.moe_route(xd, dev(router), used)
    dwg, dwu, dwd = dev_weights(wg), dev_weights(wu), dev_weights(wd)
    outs = []
    for path in (aotx_b200.PATH_TENSOR, aotx_b200.PATH_GENERAL):
        ctx.set_path(path)
        try:
            outs.append(ctx.moe_ffn(dwg, dwu, dwd, experts, hidden, ffn, xd, prob, ids).cpu().numpy())
        finally:
            ctx.set_path(0)
    torch.cuda.synchronize()
    a, b = outs
    assert np.isfinite(a).all()
    assert np.abs(a - b).max() <= 1e-2 * np.abs(b).max() + 1e-3
    counts = np.bincount(ids.cpu().numpy().reshape(-1), minlength=experts)
    assert counts.sum() == tokens * used and counts.max() > 32
    assert ctx.device_status() == 0
