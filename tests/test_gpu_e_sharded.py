"""The sharded paths on real GPUs (needs two): every rank's result equals the single-GPU
result of the same library to float rounding, and the oracle's within the product bound."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    import aotx_b200
    from aotx_b200.sharded import (ColumnSplit, column_split_on_gpu, expert_parallel_on_gpu, shard_rows)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    ctx = aotx_b200.Q8Context(rank)
    ok = True
    # column split
    n, k, m = 3000, 1024, 9
    w = aotx_b200.synth_q8_0(n, k, 5)
    x = torch.from_numpy(np.random.Generator(np.random.PCG64(6)).standard_normal((m, k)).astype(np.float16)).cuda()
    b0, b1 = ColumnSplit.shard_bytes(n, k, world, rank)
    w_all = torch.from_numpy(w).cuda()
    w_local = torch.from_numpy(w[b0:b1].copy()).cuda()
    split = column_split_on_gpu(ctx, w_local, n, k, world, rank)
    y = split.matmul(x, m)
    want = ctx.matmul(w_all, n, k, x)
    torch.cuda.synchronize()
    # a different split of the rows changes where tiles are cut between blocks, hence the
    # order of a few float additions: equal to float rounding, not bit for bit
    ok = ok and bool((y - want).abs().max() <= 1e-4 * want.abs().max())
    from oracle.binding import Oracle
    oracle = Oracle()
    x_bits = x.cpu().numpy().view(np.uint16)
    ok = ok and oracle.diff(y.cpu().numpy(), oracle.product(w, n, k, x_bits, m))[0] == 0
    # the same split with the gather fused into the product's stores (symmetric memory)
    from aotx_b200.sharded import ColumnSplitFused
    nf, kf = 3072, 1024
    wf = aotx_b200.synth_q8_0(nf, kf, 15)
    f0, f1 = ColumnSplit.shard_bytes(nf, kf, world, rank)
    fused = ColumnSplitFused(ctx, torch.from_numpy(wf[f0:f1].copy()).cuda(), nf, kf, world, rank, 16,
                             torch.float32)
    xf = x[:, :kf].contiguous()
    for _ in range(2):
        yf = fused.matmul(xf, m)
    wantf = ctx.matmul(torch.from_numpy(wf).cuda(), nf, kf, xf)
    torch.cuda.synchronize()
    ok = ok and bool((yf - wantf).abs().max() <= 1e-4 * wantf.abs().max())
    ok = ok and oracle.diff(yf.cpu().numpy(), oracle.product(wf, nf, kf, np.ascontiguousarray(x_bits[:, :kf]), m))[0] == 0
    # expert parallel
    experts, used, hidden, ffn, tokens_all = 16, 4, 512, 256, 40
    wg = aotx_b200.synth_q8_0(experts * ffn, hidden, 1)
    wu = aotx_b200.synth_q8_0(experts * ffn, hidden, 2)
    wd = aotx_b200.synth_q8_0(experts * hidden, ffn, 3)
    rng = np.random.Generator(np.random.PCG64(4))
    x_all = torch.from_numpy(rng.standard_normal((tokens_all, hidden)).astype(np.float16)).cuda()
    router = torch.from_numpy((rng.standard_normal((experts, hidden)) / np.sqrt(hidden)).astype(np.float32)).cuda()
    prob, ids = ctx.moe_route(x_all, router, used)
    full = ctx.moe_ffn(torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda(), torch.from_numpy(wd).cuda(),
                       experts, hidden, ffn, x_all, prob, ids)
    e0, e1 = shard_rows(experts, world, rank)
    t0, t1 = shard_rows(tokens_all, world, rank)
    sg, sd = ffn * (hidden // 32) * 34, hidden * (ffn // 32) * 34
    ep = expert_parallel_on_gpu(ctx, torch.from_numpy(wg[e0 * sg:e1 * sg].copy()).cuda(),
                                torch.from_numpy(wu[e0 * sg:e1 * sg].copy()).cuda(),
                                torch.from_numpy(wd[e0 * sd:e1 * sd].copy()).cuda(), experts, used, hidden,
                                ffn, world, rank)
    out = ep.ffn(x_all[t0:t1].contiguous(), prob[t0:t1].contiguous(), ids[t0:t1].contiguous())
    torch.cuda.synchronize()
    ok = ok and bool((out - full[t0:t1]).abs().max() <= 1e-4 * full.abs().max())
    want_moe = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x_all[t0:t1].cpu().numpy().view(np.uint16),
                              prob[t0:t1].cpu().numpy(), ids[t0:t1].cpu().numpy().view(np.uint32))
    ok = ok and oracle.within_bound(out.cpu().numpy(), want_moe.astype(np.float64))[0]
    # the same step with the exchange folded into the library's kernels (aotx_q8_moe_ep), three
    # steps in a row over two sets of inputs (the buffers are reused from step to step)
    from aotx_b200.sharded import ExpertParallelFused
    fused_ep = ExpertParallelFused(ctx, torch.from_numpy(wg[e0 * sg:e1 * sg].copy()).cuda(),
                                   torch.from_numpy(wu[e0 * sg:e1 * sg].copy()).cuda(),
                                   torch.from_numpy(wd[e0 * sd:e1 * sd].copy()).cuda(), experts, used, hidden,
                                   ffn, world, rank, t1 - t0)
    x_other = (x_all * 0.5).contiguous()
    prob_o, ids_o = ctx.moe_route(x_other, router, used)
    full_o = ctx.moe_ffn(torch.from_numpy(wg).cuda(), torch.from_numpy(wu).cuda(), torch.from_numpy(wd).cuda(),
                         experts, hidden, ffn, x_other, prob_o, ids_o)
    for xs, ps, sel, want_full in ((x_all, prob, ids, full), (x_other, prob_o, ids_o, full_o),
                                   (x_all, prob, ids, full)):
        got = fused_ep.ffn(xs[t0:t1].contiguous(), ps[t0:t1].contiguous(), sel[t0:t1].contiguous()).clone()
        torch.cuda.synchronize()
        ok = ok and bool((got - want_full[t0:t1]).abs().max() <= 1e-4 * want_full.abs().max())
    ok = ok and oracle.within_bound(got.cpu().numpy(), want_moe.astype(np.float64))[0]
    ok = ok and ctx.device_status() == 0
    result[rank] = ok
    dist.destroy_process_group()


def test_column_split_and_expert_parallel_on_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_worker, args=(2, _free_port(), result), nprocs=2, join=True)
    assert dict(result) == {0: True, 1: True}
