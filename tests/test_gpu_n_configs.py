"""Every shape of the benchmark's configurations that the other files do not reach, against the
oracle: the prefill layer at 2048 rows in bfloat16, the large projections of the sharded
configuration on one device, and repeat-and-compare probes of every shape class that is only
sampled.  Sampled checks use the reference's spot measure (tests/matrix_test.cu:279-312); one
slice of each prefill projection is compared in full."""
import numpy as np
import pytest

from _util import check_columns, check_product, dev, dev_weights, device_synth_q8_0, torch_mod, x_bf16_bits
from oracle.binding import row_bytes

pytestmark = pytest.mark.gpu

LAYER = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]


@pytest.fixture(scope="module")
def ctx():
    import aotx_b200
    c = aotx_b200.Q8Context(0)
    yield c
    assert c.device_status() == 0
    c.close()


def _slice_compare(oracle, w_host, n, k, bits, m, y, first, rows):
    """The whole product on weight rows [first, first + rows) against the oracle."""
    piece = w_host[first * row_bytes(k):(first + rows) * row_bytes(k)]
    want = oracle.product(piece, rows, k, bits, m, bf16=True)
    got = np.ascontiguousarray(y[:, first:first + rows])
    bad, worst = oracle.diff(got, want)
    ok, err, bound = oracle.within_bound(got, want)
    assert bad == 0, (bad, worst)
    assert ok, (err, bound)


@pytest.mark.parametrize("n,k", LAYER)
def test_prefill_layer_m2048_bf16(ctx, oracle, n, k):
    """Configuration 2: each projection of the layer at 2048 rows, bfloat16 in and out; 192 whole
    sampled columns (393 216 outputs), a full compare of 64 x-rows on a slice of 1024 weight rows,
    and the same call repeated gives the same bits.  Weights are rounded to bfloat16 on this path
    (as the activations are), so the measures are the reference's whole-product ones."""
    torch = torch_mod()
    m = 2048
    w = device_synth_q8_0(n, k, n + k + 2)
    x, bits = x_bf16_bits(m, k, 21)
    xd = x.cuda()
    y = ctx.matmul(w, n, k, xd, y_dtype=torch.bfloat16)
    again = ctx.matmul(w, n, k, xd, y_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert torch.equal(y, again)
    w_host = w.cpu().numpy()
    got = y.float().cpu().numpy()
    check_columns(oracle, w_host, n, k, bits, m, got)
    first = (n // 2 // 128) * 128 - 64          # straddles two row tiles
    rows_x = np.arange(m - 64, m)
    _slice_compare(oracle, w_host, n, k, np.ascontiguousarray(bits[rows_x]), 64,
                   np.ascontiguousarray(got[rows_x]), first, 1024)


@pytest.mark.parametrize("m", [1, 8, 64])
def test_lm_head_8192_to_151936(ctx, oracle, m):
    """Configuration 4, LM head on one device."""
    torch = torch_mod()
    n, k = 151936, 8192
    w = device_synth_q8_0(n, k, 70 + m)
    x, bits = x_bf16_bits(m, k, 22 + m)
    xd = x.cuda()
    y = ctx.matmul(w, n, k, xd, y_dtype=torch.float32)
    again = ctx.matmul(w, n, k, xd, y_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(y, again)
    got = y.cpu().numpy()
    w_host = w.cpu().numpy()
    check_product(oracle, w_host, n, k, bits, m, got, bf16=True, full_limit=0, spots=4096)
    _slice_compare(oracle, w_host, n, k, bits, m, got, n - 1000, 1000)   # the ragged last tiles


@pytest.mark.parametrize("n,k", [(57344, 8192), (8192, 28672)])
@pytest.mark.parametrize("m", [1, 32, 2048])
def test_llama70b_ffn_projections(ctx, oracle, n, k, m):
    """Configuration 4, the 70B-shaped gate+up and down projections on one device."""
    torch = torch_mod()
    w = device_synth_q8_0(n, k, n + m)
    x, bits = x_bf16_bits(m, k, 23 + m)
    xd = x.cuda()
    y = ctx.matmul(w, n, k, xd, y_dtype=torch.float32)
    again = ctx.matmul(w, n, k, xd, y_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(y, again)
    got = y.cpu().numpy()
    w_host = w.cpu().numpy()
    if m > 128:
        check_columns(oracle, w_host, n, k, bits, m, got, columns=64)
    else:
        check_product(oracle, w_host, n, k, bits, m, got, bf16=True, full_limit=0, spots=4096)
    rows_x = np.arange(max(0, m - 32), m)
    _slice_compare(oracle, w_host, n, k, np.ascontiguousarray(bits[rows_x]), len(rows_x),
                   np.ascontiguousarray(got[rows_x]), n // 2 - 64, 512)


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 1), (6144, 4096, 32), (28672, 4096, 32), (4096, 14336, 32),
                                   (28672, 4096, 64), (4096, 14336, 128)])
def test_repeats_of_the_decode_shapes(ctx, n, k, m):
    torch = torch_mod()
    w = device_synth_q8_0(n, k, 8)
    x, _ = x_bf16_bits(m, k, 9)
    xd = x.cuda()
    outs = [ctx.matmul(w, n, k, xd) for _ in range(6)]
    torch.cuda.synchronize()
    for other in outs[1:]:
        assert torch.equal(other, outs[0])
