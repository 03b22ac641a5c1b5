"""Dequantisation on the device: bit-exact against the oracle and the golden fixtures
(cases of tests/matrix_test.cu:347-378 and larger ones)."""
import numpy as np
import pytest

from _util import dev, dev_weights, torch_mod

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import aotx_b200
    c = aotx_b200.Q8Context(0)
    yield c
    c.close()


def test_golden_rows(ctx, golden):
    torch = torch_mod()
    w = dev_weights(golden["dequant_w"])
    for rows in (1, 64):
        out = ctx.dequant(w, 256, 16, rows)
        torch.cuda.synchronize()
        got = out.view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(got, golden["dequant_want"][16:16 + rows])


def test_benchmark_distribution_with_subnormal_scales(ctx, oracle):
    import aotx_b200
    torch = torch_mod()
    n, k = 257, 4096
    w_host = aotx_b200.synth_q8_0(n, k, 21)
    w = dev_weights(w_host)
    out = ctx.dequant(w, k, 0, n)
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle.dequant(w_host, k, 0, n)
    assert np.array_equal(got, want)
    q, d = aotx_b200.unpack_q8_0(w_host, n, k)
    assert (d.astype(np.float32) < 6.1e-5).mean() > 0.1
    # subnormal results must be kept, not flushed
    sub = (np.abs(want.view(np.float16).astype(np.float32)) < 6.1e-5) & (want.view(np.float16) != 0)
    assert sub.any()


def test_every_scale_and_byte(ctx, oracle):
    """All 256 byte values against a sweep of scales, including the smallest halves."""
    import aotx_b200
    torch = torch_mod()
    scales = np.concatenate([np.arange(0, 2048, 7), np.arange(2048, 0x7C00, 53)]).astype(np.uint16)
    n = scales.size
    k = 256
    q = np.tile(np.arange(-128, 128, dtype=np.int16).astype(np.int8), (n, 1))
    d = np.repeat(scales.view(np.float16)[:, None], k // 32, axis=1)
    w_host = aotx_b200.pack_q8_0(q, d)
    out = ctx.dequant(dev_weights(w_host), k, 0, n)
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, oracle.dequant(w_host, k, 0, n))


def test_whole_projection(ctx, oracle):
    """A whole 4096 x 4096 tensor of the benchmark's distribution, 16.8 M values, bit for bit."""
    import aotx_b200
    torch = torch_mod()
    n = k = 4096
    w_host = aotx_b200.synth_q8_0(n, k, 33)
    out = ctx.dequant(dev_weights(w_host), k, 0, n)
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, oracle.dequant(w_host, k, 0, n))


def test_row_window_and_unaligned_output(ctx, oracle):
    import aotx_b200
    torch = torch_mod()
    n, k = 40, 96
    w_host = aotx_b200.synth_q8_0(n, k, 5)
    w = dev_weights(w_host)
    buf = torch.full((7 * k + 2 + 8,), -1.0, dtype=torch.float16, device="cuda")
    out = buf[2:2 + 7 * k].view(7, k)  # 4-byte aligned only
    ctx.dequant(w, k, 11, 7, out=out)
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, oracle.dequant(w_host, k, 11, 7))
    assert (buf[:2] == -1).all() and (buf[2 + 7 * k:] == -1).all()


def test_wrong_type_writes_nothing(ctx):
    import aotx_b200
    torch = torch_mod()
    w = dev_weights(aotx_b200.synth_q8_0(4, 64, 1))
    out = torch.full((4, 64), 3.0, dtype=torch.float16, device="cuda")
    with pytest.raises(aotx_b200.Q8Error) as err:
        ctx.dequant(w, 64, 0, 4, out=out, type=9)  # Q8_1: no layout here, nor in the reference
    assert err.value.code == 2
    assert (out == 3.0).all()
