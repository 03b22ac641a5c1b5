"""The expert-parallel entry (aotx_q8_moe_ep) on one GPU: with one rank it is the single-GPU
step (same tables, same schedule, the same floats).  The two-GPU run is
tests/test_gpu_e_sharded.py."""
import numpy as np
import pytest

from _util import torch_mod

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import aotx_b200
    c = aotx_b200.Q8Context(0)
    yield c
    c.close()


def _case(torch, ctx, experts, used, hidden, ffn, tokens, seed):
    import aotx_b200
    w = [aotx_b200.synth_q8_0(experts * rows, k, seed + i)
         for i, (rows, k) in enumerate(((ffn, hidden), (ffn, hidden), (hidden, ffn)))]
    rng = np.random.Generator(np.random.PCG64(seed))
    x = torch.from_numpy(rng.standard_normal((tokens, hidden)).astype(np.float16)).cuda()
    router = torch.from_numpy((rng.standard_normal((experts, hidden)) / np.sqrt(hidden)).astype(np.float32)).cuda()
    prob, ids = ctx.moe_route(x, router, used)
    return w, x, prob, ids


@pytest.mark.parametrize("experts,used,hidden,ffn,tokens", [(16, 4, 512, 256, 40), (8, 2, 256, 768, 70)])
def test_one_rank_is_the_single_gpu_step(ctx, oracle, experts, used, hidden, ffn, tokens):
    torch = torch_mod()
    w, x, prob, ids = _case(torch, ctx, experts, used, hidden, ffn, tokens, 31)
    wd = [torch.from_numpy(t).cuda() for t in w]
    proj = torch.zeros((tokens * used, hidden), dtype=torch.float32, device="cuda")
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty((tokens, hidden), dtype=torch.float32, device="cuda")
    work = ctx.moe_ep_workspace(tokens, used, hidden, ffn, 1)

    def run(sel):
        ctx.moe_ep(*wd, experts, hidden, ffn, [x.data_ptr()], [sel.data_ptr()], prob, tokens, used,
                   [proj.data_ptr()], [flags.data_ptr()], 0, step, out, work)
        torch.cuda.synchronize()
        return out.clone()

    want = ctx.moe_ffn(*wd, experts, hidden, ffn, x, prob, ids)
    got = run(ids)
    assert torch.equal(got, want)
    ref = oracle.moe_ffn(*w, experts, hidden, ffn, x.cpu().numpy().view(np.uint16), prob.cpu().numpy(),
                         ids.cpu().numpy().view(np.uint32))
    assert oracle.within_bound(got.cpu().numpy(), ref.astype(np.float64))[0]
    # a selection that names no expert is left out, here as in the single-GPU step
    bad = ids.clone()
    bad[3, 0] = experts + 5
    assert torch.equal(run(bad), ctx.moe_ffn(*wd, experts, hidden, ffn, x, prob, bad))
    assert ctx.device_status() == 0
    assert int(step.item()) == 4                 # two barriers a call


def test_argument_checks(ctx):
    torch = torch_mod()
    lib = ctx.lib
    import ctypes as C
    one = (C.c_void_p * 1)(C.c_void_p(256))
    code = lib.aotx_q8_moe_ep(ctx.handle, None, 256, 256, 256, 8, 16, 512, 256, one, one, 256, 4, 2, one, one, 1, 1,
                              256, 256, 0, 256, 1 << 30)
    assert code != 0                              # rank >= peers
    code = lib.aotx_q8_moe_ep(ctx.handle, None, 256, 256, 256, 8, 16, 512, 256, one, one, 256, 4, 2, one, one, 1, 0,
                              256, 256, 0, 256, 16)
    assert code != 0                              # workspace too small
    assert lib.aotx_q8_moe_ep_workspace_bytes(4, 2, 512, 256, 9) == 0
