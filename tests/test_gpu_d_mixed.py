"""bfloat16 activations through both kernel families, and the benchmark's decode and prefill
shapes."""
import numpy as np
import pytest

from _util import GUARD, check_product, dev, dev_weights, torch_mod, x_bf16_bits, x_fp16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import aotx_b200
    c = aotx_b200.Q8Context(0)
    yield c
    assert c.device_status() == 0
    c.close()


@pytest.mark.parametrize("path_name", ["PATH_GENERAL", "PATH_TENSOR"])
@pytest.mark.parametrize("n,k,m", [(256, 512, 1), (640, 1024, 32), (512, 768, 130), (384, 1024, 300)])
def test_bf16_activations(ctx, oracle, path_name, n, k, m):
    import aotx_b200
    torch = torch_mod()
    w = aotx_b200.synth_q8_0(n, k, 500 + m)
    x, bits = x_bf16_bits(m, k, 31 + m)
    ctx.set_path(getattr(aotx_b200, path_name))
    y = torch.full((m + 1, n), GUARD, dtype=torch.bfloat16, device="cuda")
    try:
        ctx.matmul(dev_weights(w), n, k, x.cuda(), y=y[:m])
        torch.cuda.synchronize()
    finally:
        ctx.set_path(0)
    got = y.float().cpu().numpy()
    want = oracle.product(w, n, k, bits, m, bf16=True)
    ok, err, bound = oracle.within_bound(got[:m], want)
    assert ok, (err, bound)
    assert (got[m:] == float(torch.tensor(GUARD).to(torch.bfloat16))).all()


@pytest.mark.parametrize("n,k", [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)])
def test_decode_layer_shapes_m32(ctx, oracle, n, k):
    """The four projections of the benchmark's decode layer at 32 rows, bf16 in and out."""
    import aotx_b200
    torch = torch_mod()
    m = 32
    w = aotx_b200.synth_q8_0(n, k, n + k)
    x, bits = x_bf16_bits(m, k, 3)
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    ctx.matmul(dev_weights(w), n, k, x.cuda(), y=y)
    torch.cuda.synchronize()
    check_product(oracle, w, n, k, bits, m, y.cpu().numpy(), bf16=True)


def test_prefill_shape_m2048_spot(ctx, oracle):
    import aotx_b200
    torch = torch_mod()
    n, k, m = 4096, 4096, 2048
    w = aotx_b200.synth_q8_0(n, k, 8)
    x = x_fp16(m, k, 4)
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    ctx.matmul(dev_weights(w), n, k, dev(x), y=y)
    torch.cuda.synchronize()
    check_product(oracle, w, n, k, x.view(np.uint16), m, y.cpu().numpy(), full_limit=0, spots=2048)


@pytest.mark.parametrize("n,k,m", [(1280, 512, 700), (2560, 256, 2048), (2432, 768, 1100)])
def test_wide_batches_full_compare(ctx, oracle, n, k, m):
    """Batches above 128 rows (the 256-row kernel): fewer tiles than SMs, one whole wave plus a
    cut tail, and a ragged last token tile, each against the whole oracle product."""
    import aotx_b200
    torch = torch_mod()
    w = aotx_b200.synth_q8_0(n, k, n + m)
    x = x_fp16(m, k, m)
    y = torch.full((m + 1, n), GUARD, dtype=torch.float32, device="cuda")
    ctx.matmul(dev_weights(w), n, k, dev(x), y=y[:m])
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    check_product(oracle, w, n, k, x.view(np.uint16), m, got[:m])
    assert (got[m:] == GUARD).all()


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 32), (4736, 4096, 300), (4096, 4096, 2048)])
def test_repeated_launches_are_bit_identical(ctx, n, k, m):
    """The sums run in a fixed order (tiles cut between blocks are added in block order), so
    the same call gives the same bits every time; a difference means a race."""
    import aotx_b200
    torch = torch_mod()
    w = dev_weights(aotx_b200.synth_q8_0(n, k, 8))
    x = dev(x_fp16(m, k, 9))
    outs = [ctx.matmul(w, n, k, x) for _ in range(6)]
    torch.cuda.synchronize()
    for other in outs[1:]:
        assert torch.equal(other, outs[0])


def test_linearity_at_full_size(ctx):
    """A size-independent property at the benchmark's largest decode shape: the product is
    linear in x, so y(x1 + x2) = y(x1) + y(x2) to float rounding when the sums of inputs are
    exact in half."""
    import aotx_b200
    torch = torch_mod()
    n, k, m = 28672, 4096, 32
    w = dev_weights(aotx_b200.synth_q8_0(n, k, 1))
    rng = np.random.Generator(np.random.PCG64(12))
    a = (rng.integers(-64, 64, (m, k)) / 32.0).astype(np.float16)
    b = (rng.integers(-64, 64, (m, k)) / 32.0).astype(np.float16)
    ya = ctx.matmul(w, n, k, dev(a))
    yb = ctx.matmul(w, n, k, dev(b))
    yab = ctx.matmul(w, n, k, dev((a + b).astype(np.float16)))
    torch.cuda.synchronize()
    scale = float(yab.abs().max())
    assert float((ya + yb - yab).abs().max()) <= 1e-5 * scale + 1e-9
