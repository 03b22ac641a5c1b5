"""The products with the next step of the layer folded into their store
(aotx_q8_matmul_fused, aotx_q8_moe_ffn_fused) against the two-step forms.

Residual add: the fused call forms the same float sums as the plain product on the same shape
and adds each once, so it must equal `y0 + product` bit for bit (the reference's
aotx_model_residual is that one float add, cuda/model/norm.cu:78-89).  Gated unit: gate and
up rows are interleaved in one tensor; the result must equal half(silu(gate) * up) formed from
the separate products up to the float summation order (a binary16 rounding step), and the
routed-expert step built on it must match the oracle like the unfused one."""
import numpy as np
import pytest

from _util import GUARD, dev, dev_weights, torch_mod, x_fp16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import aotx_b200
    c = aotx_b200.Q8Context(0)
    yield c
    assert c.device_status() == 0
    c.close()


# (n, k, m): general kernel (rows of 136 bytes), one token tile, several token tiles, cut tiles
SHAPES = [(80, 128, 3), (384, 512, 1), (640, 1024, 32), (512, 768, 130), (4096, 4096, 32), (256, 1024, 300)]


@pytest.mark.parametrize("n,k,m", SHAPES)
def test_residual_add_equals_product_then_add(ctx, n, k, m):
    import aotx_b200
    torch = torch_mod()
    w = dev_weights(aotx_b200.synth_q8_0(n, k, 60 + m))
    x = dev(x_fp16(m, k, 61 + m))
    rng = np.random.Generator(np.random.PCG64(62 + m))
    y0 = dev(rng.standard_normal((m + 2, n)).astype(np.float32))
    y0[m:] = GUARD
    plain = ctx.matmul(w, n, k, x)
    y = y0.clone()
    ctx.matmul_fused(w, n, k, x, aotx_b200.EPILOGUE_ADD, m=m, y=y[:m])
    torch.cuda.synchronize()
    assert torch.equal(y[:m], y0[:m] + plain)
    assert bool((y[m:] == GUARD).all())
    # twice: the stream accumulates
    ctx.matmul_fused(w, n, k, x, aotx_b200.EPILOGUE_ADD, m=m, y=y[:m])
    torch.cuda.synchronize()
    assert torch.equal(y[:m], (y0[:m] + plain) + plain)


def test_residual_add_with_a_live_batch_word(ctx):
    import aotx_b200
    torch = torch_mod()
    n, k, m = 512, 1024, 32
    w = dev_weights(aotx_b200.synth_q8_0(n, k, 70))
    x = dev(x_fp16(m, k, 71))
    live = torch.tensor([5], dtype=torch.int32, device="cuda")
    y = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    ctx.matmul_fused(w, n, k, x, aotx_b200.EPILOGUE_ADD, m=m, m_dev=live, y=y)
    plain = ctx.matmul(w, n, k, x)
    torch.cuda.synchronize()
    assert torch.equal(y[:5], plain[:5])
    assert bool((y[5:] == 0).all())


@pytest.mark.parametrize("half_n,k,m", [(40, 128, 3), (192, 512, 1), (320, 1024, 32), (256, 768, 130),
                                        (14336, 4096, 32), (128, 1024, 300)])
@pytest.mark.parametrize("out", ["float16", "float32"])
def test_gated_unit_equals_two_products_then_swiglu(ctx, oracle, half_n, k, m, out):
    import aotx_b200
    torch = torch_mod()
    wg = aotx_b200.synth_q8_0(half_n, k, 80 + m)
    wu = aotx_b200.synth_q8_0(half_n, k, 81 + m)
    both = dev_weights(aotx_b200.interleave_rows(wg, wu, k))
    # activations large enough that silu is not in its linear part everywhere
    x = dev((x_fp16(m, k, 82 + m).astype(np.float32) * 8.0).astype(np.float16))
    gate = ctx.matmul(dev_weights(wg), half_n, k, x)
    up = ctx.matmul(dev_weights(wu), half_n, k, x)
    dtype = getattr(torch, out)
    y = torch.full((m + 1, half_n), GUARD, dtype=dtype, device="cuda")
    ctx.matmul_fused(both, 2 * half_n, k, x, aotx_b200.EPILOGUE_SWIGLU, m=m, y=y[:m])
    torch.cuda.synchronize()
    want = (gate / (1.0 + torch.exp(-gate))) * up
    got = y[:m].float()
    scale = float(want.abs().max())
    step = 2.0 ** -9 if out == "float16" else 2.0 ** -18
    assert bool(torch.isfinite(got).all())
    assert bool(((got - want).abs() <= step * want.abs() + 1e-5 * scale + 1e-7).all())
    assert bool((y[m:].float() == float(torch.tensor(GUARD).to(dtype))).all())
    if float(m) * half_n * k <= 2e9:
        # and against the oracle's double products, independent of the library's plain kernels
        bits = x.cpu().numpy().view(np.uint16)
        g = oracle.product(wg, half_n, k, bits, m)
        u = oracle.product(wu, half_n, k, bits, m)
        ideal = g / (1.0 + np.exp(-g)) * u
        # the reference's measure (the general kernel multiplies with unrounded weights, the
        # oracle with the half-rounded ones, as for the plain product)
        assert oracle.diff(got.cpu().numpy(), ideal)[0] == 0


def test_fused_arguments(ctx):
    import aotx_b200
    from aotx_b200.q8 import Q8Error
    torch = torch_mod()
    n, k, m = 256, 512, 4
    w = dev_weights(aotx_b200.synth_q8_0(n, k, 1))
    x = dev(x_fp16(m, k, 2))
    with pytest.raises(Q8Error):   # the residual stream is float
        ctx.matmul_fused(w, n, k, x, aotx_b200.EPILOGUE_ADD, y=torch.zeros((m, n), dtype=torch.float16, device="cuda"))
    with pytest.raises(Q8Error):   # pairs of rows
        ctx.matmul_fused(w, n - 1, k, x, aotx_b200.EPILOGUE_SWIGLU)
    with pytest.raises(Q8Error):
        ctx.matmul_fused(w, n, k, x, 3)
    plain = ctx.matmul(w, n, k, x)
    same = ctx.matmul_fused(w, n, k, x, aotx_b200.EPILOGUE_STORE)
    torch.cuda.synchronize()
    assert torch.equal(plain, same)


@pytest.mark.parametrize("tokens,experts,used,hidden,ffn", [(64, 5, 3, 512, 256), (200, 7, 2, 512, 256),
                                                            (64, 128, 8, 2048, 768), (512, 32, 4, 1024, 512)])
def test_routed_experts_with_interleaved_gate_up(ctx, oracle, tokens, experts, used, hidden, ffn):
    import aotx_b200
    torch = torch_mod()
    rng = np.random.Generator(np.random.PCG64(90 + tokens))
    wg = aotx_b200.synth_q8_0(experts * ffn, hidden, 91)
    wu = aotx_b200.synth_q8_0(experts * ffn, hidden, 92)
    wd = aotx_b200.synth_q8_0(experts * hidden, ffn, 93)
    x = rng.standard_normal((tokens, hidden)).astype(np.float16)
    router = rng.standard_normal((experts, hidden)).astype(np.float32) / np.float32(np.sqrt(hidden))
    xd = dev(x)
    prob, ids = ctx.moe_route(xd, dev(router), used)
    dwd = dev_weights(wd)
    both = dev_weights(aotx_b200.interleave_rows(wg, wu, hidden, groups=experts))
    out = torch.full((tokens + 2, hidden), GUARD, dtype=torch.float32, device="cuda")
    ctx.moe_ffn_fused(both, dwd, experts, hidden, ffn, xd, prob, ids, tokens=tokens, out=out[:tokens])
    plain = ctx.moe_ffn(dev_weights(wg), dev_weights(wu), dwd, experts, hidden, ffn, xd, prob, ids)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert (got[tokens:] == GUARD).all()
    ref = plain.cpu().numpy()
    assert np.abs(got[:tokens] - ref).max() <= 1e-2 * np.abs(ref).max() + 1e-6
    if tokens * experts <= 64 * 128:
        want = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x.view(np.uint16), prob.cpu().numpy(),
                              ids.cpu().numpy().view(np.uint32))
        ok, err, bound = oracle.within_bound(got[:tokens], want.astype(np.float64))
        assert ok, (err, bound)
