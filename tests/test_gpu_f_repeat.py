"""Repeat-and-compare probes: every sum in this library runs in a fixed order, so one call
repeated on the same inputs must give the same bits.  A difference means a race between the
warps of a block or between blocks, which a tolerance test against the oracle can miss.
(The fp16 product shapes are probed in test_gpu_d_mixed.py.)"""
import numpy as np
import pytest

from _util import dev, dev_weights, torch_mod, x_bf16_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import aotx_b200
    c = aotx_b200.Q8Context(0)
    yield c
    assert c.device_status() == 0
    c.close()


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 32), (6144, 4096, 64), (4736, 4096, 300)])
def test_bf16_product_repeats_bit_identically(ctx, n, k, m):
    """bfloat16 activations are turned into binary16 in shared memory by the converter warps
    before the MMA reads them: one more hand-over than the fp16 case has."""
    import aotx_b200
    torch = torch_mod()
    w = dev_weights(aotx_b200.synth_q8_0(n, k, 18))
    x, _ = x_bf16_bits(m, k, 19)
    xd = x.cuda()
    outs = [ctx.matmul(w, n, k, xd, y_dtype=torch.bfloat16) for _ in range(6)]
    torch.cuda.synchronize()
    for other in outs[1:]:
        assert torch.equal(other, outs[0])


@pytest.mark.parametrize("x_name", ["bfloat16", "float16"])
def test_prefill_kernel_repeats_bit_identically_many_times(ctx, x_name):
    """Sixty launches of the prefill kernel at 28672 x 4096 x 2048.  This is the probe that
    caught a raw stage handed back to the copying thread before a warp's shared-memory loads
    had returned: about one launch in forty had one weight row of one tile wrong, bfloat16
    only.  Six launches, as above, would have passed nine times in ten."""
    from _util import device_synth_q8_0
    torch = torch_mod()
    n, k, m = 28672, 4096, 2048
    w = device_synth_q8_0(n, k, 77)
    xd = torch.randn(m, k, device="cuda").to(getattr(torch, x_name))
    first = ctx.matmul(w, n, k, xd, y_dtype=torch.float32)
    for _ in range(6):
        outs = [ctx.matmul(w, n, k, xd, y_dtype=torch.float32) for _ in range(10)]
        torch.cuda.synchronize()
        for other in outs:
            assert torch.equal(other, first)
        del outs


@pytest.mark.parametrize("m,x_name", [(64, "bfloat16"), (128, "bfloat16"), (100, "float16")])
def test_mid_batch_kernel_repeats_bit_identically_many_times(ctx, m, x_name):
    """Forty launches of the one-block-per-SM kernel at 28672 x 4096 (row-wise stores through
    the warps' staging buffers; bfloat16 x turned into binary16 by the pass before the product)."""
    from _util import device_synth_q8_0
    torch = torch_mod()
    n, k = 28672, 4096
    w = device_synth_q8_0(n, k, 78)
    xd = torch.randn(m, k, device="cuda").to(getattr(torch, x_name))
    first = ctx.matmul(w, n, k, xd, y_dtype=torch.bfloat16)
    for _ in range(2):
        outs = [ctx.matmul(w, n, k, xd, y_dtype=torch.bfloat16) for _ in range(20)]
        torch.cuda.synchronize()
        for other in outs:
            assert torch.equal(other, first)
        del outs


def test_routed_experts_repeat_bit_identically(ctx):
    """Grouped mode (tile table, scattered stores) on a shape where most experts are hit."""
    import aotx_b200
    torch = torch_mod()
    tokens, experts, used, hidden, ffn = 256, 32, 4, 1024, 512
    rng = np.random.Generator(np.random.PCG64(77))
    wg = dev_weights(aotx_b200.synth_q8_0(experts * ffn, hidden, 71))
    wu = dev_weights(aotx_b200.synth_q8_0(experts * ffn, hidden, 72))
    wd = dev_weights(aotx_b200.synth_q8_0(experts * hidden, ffn, 73))
    x = dev(rng.standard_normal((tokens, hidden)).astype(np.float16))
    router = dev(rng.standard_normal((experts, hidden)).astype(np.float32) / np.float32(np.sqrt(hidden)))
    prob, ids = ctx.moe_route(x, router, used)
    outs = [ctx.moe_ffn(wg, wu, wd, experts, hidden, ffn, x, prob, ids).clone() for _ in range(30)]
    torch.cuda.synchronize()
    for other in outs[1:]:
        assert torch.equal(other, outs[0])
    # the interleaved form (gated unit in the row-wise store of the gate+up product)
    both = dev_weights(aotx_b200.interleave_rows(aotx_b200.synth_q8_0(experts * ffn, hidden, 71),
                                                 aotx_b200.synth_q8_0(experts * ffn, hidden, 72), hidden,
                                                 groups=experts))
    outs = [ctx.moe_ffn_fused(both, wd, experts, hidden, ffn, x, prob, ids).clone() for _ in range(30)]
    torch.cuda.synchronize()
    for other in outs[1:]:
        assert torch.equal(other, outs[0])
