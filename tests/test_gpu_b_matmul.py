"""The product on the device against the oracle: the reference's own cases
(tests/matrix_test.cu:382-468, tests/embedded_modules_test.cu:22-51) through both kernel
families, then the benchmark's shapes."""
import numpy as np
import pytest

from _util import GUARD, check_product, dev, dev_weights, torch_mod, x_fp16
from oracle.binding import SEED

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import aotx_b200
    c = aotx_b200.Q8Context(0)
    yield c
    assert c.device_status() == 0
    c.close()


def _run(ctx, w_host, n, k, x_host, m, y_dtype=None, path=0, m_dev=None, rows=None):
    torch = torch_mod()
    rows = rows or m
    ctx.set_path(path)
    w = dev_weights(w_host)
    x = dev(x_host)
    y = torch.full((rows + 2, n), GUARD, dtype=y_dtype or torch.float32, device="cuda")
    ctx.matmul(w, n, k, x, m=rows, m_dev=m_dev, y=y[:rows])
    torch.cuda.synchronize()
    ctx.set_path(0)
    return y.float().cpu().numpy()


@pytest.mark.parametrize("m", [1, 64])
def test_golden_80_by_128_general(ctx, oracle, golden, m):
    """80 x 128 is no tile multiple and its rows are 136 bytes: the general kernel's shape."""
    x = golden["product_x_m%d" % m].view(np.float16)
    y = _run(ctx, golden["product_w"], 80, 128, x, m)
    want = golden["product_want_m%d" % m]
    bad, worst = oracle.diff(y[:m], want)
    assert bad == 0, worst
    assert oracle.within_bound(y[:m], want)[0]
    assert (y[m:] == GUARD).all()


def test_turned_operand_general(ctx, oracle, golden):
    y = _run(ctx, golden["turn_w"], 64, 64, golden["turn_x"].view(np.float16), 64)[:64]
    right, _ = oracle.diff(y, golden["turn_want"])
    turned, _ = oracle.diff(y, golden["turn_want_swapped"])
    assert right == 0 and turned > 0


def test_known_answer(ctx):
    """Scale 1.0, row i all i+1, x row t all t+1: y[t][i] = 32 (i+1)(t+1)."""
    torch = torch_mod()
    w = np.zeros((32, 34), np.uint8)
    w[:, 1] = 0x3C
    for i in range(32):
        w[i, 2:] = i + 1
    for m in (1, 64):
        x = np.repeat(np.arange(1, m + 1, dtype=np.float16)[:, None], 32, axis=1)
        y = _run(ctx, w.reshape(-1), 32, 32, x, m)[:m]
        want = 32.0 * np.outer(np.arange(1, m + 1), np.arange(1, 33))
        assert np.array_equal(y, want.astype(np.float32))


@pytest.mark.parametrize("n,k,m", [(128, 256, 1), (128, 256, 16), (300, 768, 5), (512, 1024, 32),
                                   (4096, 4096, 1), (1000, 2048, 64), (384, 512, 100),
                                   (256, 256, 256), (130, 512, 300), (4096, 4096, 32)])
def test_tensor_path_fp16(ctx, oracle, n, k, m):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, 100 + n + m)
    x = x_fp16(m, k, 7 + m)
    y = _run(ctx, w, n, k, x, m, path=aotx_b200.PATH_TENSOR)
    check_product(oracle, w, n, k, x.view(np.uint16), m, y[:m])
    assert (y[m:] == GUARD).all()
    assert ctx.device_status() == 0


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 1), (1000, 2048, 9), (19, 512, 3)])
def test_general_path_fp16(ctx, oracle, n, k, m):
    import aotx_b200
    w = aotx_b200.synth_q8_0(n, k, 300 + n)
    x = x_fp16(m, k, 11 + m)
    y = _run(ctx, w, n, k, x, m, path=aotx_b200.PATH_GENERAL)
    check_product(oracle, w, n, k, x.view(np.uint16), m, y[:m])
    assert (y[m:] == GUARD).all()


def test_reference_fixture_recipe_tensor_path(ctx, oracle):
    """The reference's own generator at a shape its rate cases use (2560 x 2560, m = 8;
    tests/matrix_test.cu:754-760), through the streaming kernel, spot-checked like
    tests/matrix_test.cu:279-312."""
    import aotx_b200
    n = k = 2560
    w = oracle.build(n, k, SEED + 200)
    x = oracle.input(8, k, SEED + 201)
    y = _run(ctx, w, n, k, x.view(np.float16), 8, path=aotx_b200.PATH_TENSOR)[:8]
    bad, worst = oracle.spot(w, n, k, x, 8, y, count=64)
    assert bad == 0, worst


@pytest.mark.parametrize("n,k,m", [(9728, 2560, 1), (2560, 9728, 8), (2560, 2560, 1)])
def test_reference_rate_shapes(ctx, oracle, n, k, m):
    """The other shapes of the reference's rate cases (tests/matrix_test.cu:754-760), its own
    generator, both kernel families against each other and against sampled oracle sums."""
    import aotx_b200
    w = oracle.build(n, k, SEED + 640)
    x = oracle.input(m, k, SEED + 642)
    tensor = _run(ctx, w, n, k, x.view(np.float16), m, path=aotx_b200.PATH_TENSOR)[:m]
    general = _run(ctx, w, n, k, x.view(np.float16), m, path=aotx_b200.PATH_GENERAL)[:m]
    assert oracle.spot(w, n, k, x, m, tensor, count=256)[0] == 0
    assert oracle.spot(w, n, k, x, m, general, count=256)[0] == 0
    assert np.abs(tensor - general).max() <= 1e-2 * np.abs(general).max() + 1e-3


def test_live_batch_from_device_word(ctx, oracle):
    """One call shape, several live batches: rows at and past the live batch stay as they
    were (the contract of cuda/model/product.cu:24-49)."""
    import aotx_b200
    torch = torch_mod()
    n, k, cap = 640, 1024, 64
    w = aotx_b200.synth_q8_0(n, k, 77)
    x = x_fp16(cap, k, 78)
    want = oracle.product(w, n, k, x.view(np.uint16), cap)
    for path in (aotx_b200.PATH_TENSOR, aotx_b200.PATH_GENERAL):
        for live in (0, 1, 17, 64, 200):
            word = torch.tensor([live], dtype=torch.int32, device="cuda")
            y = _run(ctx, w, n, k, x, cap, path=path, m_dev=word, rows=cap)
            rows = min(live, cap)
            if rows:
                assert oracle.diff(y[:rows], want[:rows])[0] == 0
            assert (y[rows:] == GUARD).all()


@pytest.mark.parametrize("dtype_name", ["float16", "bfloat16"])
def test_output_types(ctx, oracle, dtype_name):
    import aotx_b200
    torch = torch_mod()
    n, k, m = 512, 512, 24
    w = aotx_b200.synth_q8_0(n, k, 9)
    x = x_fp16(m, k, 10)
    want = oracle.product(w, n, k, x.view(np.uint16), m)
    for path in (aotx_b200.PATH_TENSOR, aotx_b200.PATH_GENERAL):
        dtype = getattr(torch, dtype_name)
        y = _run(ctx, w, n, k, x, m, y_dtype=dtype, path=path)
        assert oracle.within_bound(y[:m], want)[0]
        assert (y[m:] == float(torch.tensor(GUARD).to(dtype))).all()


def test_errors_write_nothing(ctx):
    import aotx_b200
    torch = torch_mod()
    w = dev_weights(aotx_b200.synth_q8_0(8, 64, 1))
    x = dev(x_fp16(2, 64, 1))
    y = torch.full((2, 8), GUARD, dtype=torch.float32, device="cuda")
    with pytest.raises(aotx_b200.Q8Error) as err:
        ctx.matmul(w, 8, 64, x, y=y, type=9)  # Q8_1: no layout here, nor in the reference
    assert err.value.code == 2
    with pytest.raises(aotx_b200.Q8Error) as err:
        ctx.matmul(w, 8, 48, x, y=y)
    assert err.value.code == 1
    ctx.set_path(aotx_b200.PATH_TENSOR)
    with pytest.raises(aotx_b200.Q8Error) as err:
        ctx.matmul(w, 8, 64, x, y=y)
    assert err.value.code == 4
    ctx.set_path(0)
    torch.cuda.synchronize()
    assert (y == GUARD).all()
