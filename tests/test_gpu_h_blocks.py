"""Every block type of the model file through aotx_q8_dequant and aotx_q8_matmul on the GPU.

The checker is the oracle's restatement of the reference's host reading (oracle/blocks_oracle.c,
pinned against the reference's own reading on the CPU by tests/test_blocks.py): the
dequantised halves must lie within the reference's acceptance bound of its doubles
(tests/matrix_kcases.h:160-190: relative error at most 2^-10 or one binary16 subnormal step),
and must equal, bit for bit, what the host build of the decoder gives; the product must match
the double product over the oracle's weights within the reference's measure
(tests/matrix_test.cu:246-274, 1e-2) and the bound max|err| <= 1e-2 max|y| + 1e-3; rows past
the batch keep their guard value; a type without a layout writes nothing
(cuda/model/dequant.cu:24-25)."""
import numpy as np
import pytest

import _blocks
from _util import GUARD, dev, dev_weights, torch_mod, x_fp16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import aotx_b200
    c = aotx_b200.Q8Context(0)
    yield c
    assert c.device_status() == 0
    c.close()


@pytest.fixture(scope="module")
def decoder(tmp_path_factory):
    return _blocks.HostDecoder(tmp_path_factory.mktemp("blocks"))


@pytest.mark.parametrize("kind", sorted(_blocks.TYPES))
def test_dequant_of_every_type_is_bit_exact(ctx, oracle, decoder, kind):
    torch = torch_mod()
    rng = np.random.default_rng(300 + kind)
    n, k = 40, 512
    w = _blocks.random_rows(kind, n, k, rng, subnormal_share=0.3)
    first, rows = 7, 29
    out = torch.full((rows + 1, k), GUARD, dtype=torch.float16, device="cuda")
    ctx.dequant(dev_weights(w), k, first, rows, out=out[:rows], type=kind)
    torch.cuda.synchronize()
    got = out.cpu().numpy().view(np.uint16)
    ideal = oracle.block_rows(kind, w, k, first, rows)
    have = got[:rows].view(np.float16).astype(np.float64)
    err = np.abs(have - ideal)
    assert np.isfinite(have).all()
    assert ((err <= np.abs(ideal) * 9.765625e-04) | (err <= 5.9604644775390625e-08)).all()
    want = decoder.rows(kind, w, n, k, half=True)[first:first + rows]
    assert np.array_equal(got[:rows], want)
    assert (got[rows:] == np.float16(GUARD).view(np.uint16)).all()


@pytest.mark.parametrize("kind", sorted(_blocks.TYPES))
@pytest.mark.parametrize("m,x_kind", [(1, "float16"), (11, "float16"), (9, "bfloat16")])
def test_product_of_every_type(ctx, oracle, decoder, kind, m, x_kind):
    torch = torch_mod()
    rng = np.random.default_rng(400 + kind + m)
    n, k = 72, 768
    w = _blocks.random_rows(kind, n, k, rng)
    weights = oracle.block_rows(kind, w, k, 0, n)
    x = torch.from_numpy(x_fp16(m, k, 500 + kind).astype(np.float32)).to(getattr(torch, x_kind))
    want = x.double().numpy() @ weights.T
    y = torch.full((m + 2, n), GUARD, dtype=torch.float32, device="cuda")
    ctx.matmul(dev_weights(w), n, k, x.cuda(), m=m, y=y[:m], type=kind)
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    assert oracle.diff(np.ascontiguousarray(got[:m]), np.ascontiguousarray(want))[0] == 0
    ok, err, bound = oracle.within_bound(np.ascontiguousarray(got[:m]), np.ascontiguousarray(want))
    assert ok, (err, bound)
    assert (got[m:] == GUARD).all()


def test_live_batch_and_half_results_on_a_k_type(ctx, oracle):
    torch = torch_mod()
    kind, n, k, m = 12, 64, 1024, 16
    rng = np.random.default_rng(9)
    w = _blocks.random_rows(kind, n, k, rng)
    weights = oracle.block_rows(kind, w, k, 0, n)
    x = x_fp16(m, k, 10)
    live = torch.tensor([5], dtype=torch.int32, device="cuda")
    y = torch.full((m, n), GUARD, dtype=torch.bfloat16, device="cuda")
    ctx.matmul(dev_weights(w), n, k, dev(x), m=m, m_dev=live, y=y, type=kind)
    torch.cuda.synchronize()
    got = y.float().cpu().numpy()
    want = x[:5].astype(np.float64) @ weights.T
    assert np.abs(got[:5] - want).max() <= 1e-2 * np.abs(want).max() + 1e-3
    assert (got[5:] == float(torch.tensor(GUARD).to(torch.bfloat16))).all()


def test_types_without_a_layout_and_rows_that_are_not_whole_blocks(ctx):
    import aotx_b200
    from aotx_b200.q8 import Q8Error
    torch = torch_mod()
    w = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    x = torch.zeros((1, 256), dtype=torch.float16, device="cuda")
    y = torch.full((1, 4), GUARD, dtype=torch.float32, device="cuda")
    for kind in (4, 5, 9, 15, 30):
        with pytest.raises(Q8Error) as info:
            ctx.matmul(w, 4, 256, x, y=y, type=kind)
        assert info.value.code == 2
    with pytest.raises(Q8Error) as info:       # a K type needs rows of whole super blocks
        ctx.matmul(w, 4, 128, x[:, :128].contiguous(), y=y, type=12)
    assert info.value.code == 1
    ctx.set_path(aotx_b200.PATH_TENSOR)
    try:
        with pytest.raises(Q8Error) as info:   # only Q8_0 has a tensor-core kernel
            ctx.matmul(w, 4, 256, x, y=y, type=12)
        assert info.value.code == 4
    finally:
        ctx.set_path(0)
    torch.cuda.synchronize()
    assert bool((y == GUARD).all())


def test_reference_q4_0_fixtures_on_the_gpu(ctx, oracle):
    """The reference's own Q4_0 cases (tests/matrix_test.cu:347-428, fixtures and expectations in
    tests/golden/reference_q4_0.npz): dequantisation of rows 16.. at 1 and 64 rows bit for bit,
    the 80 x 128 product at 1 and 64 rows of x within its measure."""
    import os
    torch = torch_mod()
    data = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_q4_0.npz"))
    w = dev_weights(data["dequant_w"])
    for rows in (1, 64):
        out = ctx.dequant(w, 256, 16, rows, type=2)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy().view(np.uint16), data["dequant_want"][16:16 + rows])
    w = dev_weights(data["product_w"])
    for m in (1, 64):
        x = dev(data["product_x_m%d" % m].view(np.float16).reshape(m, 128))
        y = torch.zeros((m, 80), dtype=torch.float32, device="cuda")
        ctx.matmul(w, 80, 128, x, y=y, type=2)
        torch.cuda.synchronize()
        assert oracle.diff(y.cpu().numpy(), data["product_want_m%d" % m])[0] == 0
