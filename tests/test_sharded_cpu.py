"""The exchange logic of the sharded paths on CPU ranks (gloo, world size 2 and 3): the local
compute step is the oracle, the collectives are real."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _column_worker(rank, world, port, n, k, m, result):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import aotx_b200
    from aotx_b200.sharded import ColumnSplit
    from oracle.binding import Oracle
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    oracle = Oracle()
    w = aotx_b200.synth_q8_0(n, k, 5)
    x = np.random.Generator(np.random.PCG64(6)).standard_normal((m, k)).astype(np.float16)
    b0, b1 = ColumnSplit.shard_bytes(n, k, world, rank)

    def product(x_t, rows):
        first, last = aotx_b200.sharded.shard_rows(n, world, rank)
        y = oracle.product(w[b0:b1], last - first, k, x_t.numpy().view(np.uint16), rows, threads=1)
        return torch.from_numpy(y.astype(np.float32))

    split = ColumnSplit(n, k, world, rank, product)
    y = split.matmul(torch.from_numpy(x), m)
    want = oracle.product(w, n, k, x.view(np.uint16), m, threads=1).astype(np.float32)
    result[rank] = bool(np.array_equal(y.numpy(), want))
    dist.destroy_process_group()


def _expert_worker(rank, world, port, bad, result):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import aotx_b200
    from aotx_b200.sharded import ExpertParallel, shard_rows
    from oracle.binding import Oracle
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    oracle = Oracle()
    experts, used, hidden, ffn, tokens_all = 7, 3, 64, 32, 12
    wg = aotx_b200.synth_q8_0(experts * ffn, hidden, 1)
    wu = aotx_b200.synth_q8_0(experts * ffn, hidden, 2)
    wd = aotx_b200.synth_q8_0(experts * hidden, ffn, 3)
    rng = np.random.Generator(np.random.PCG64(4))
    x_all = rng.standard_normal((tokens_all, hidden)).astype(np.float16)
    router = rng.standard_normal((experts, hidden)).astype(np.float32)
    prob_all, ids_all = oracle.route(x_all.view(np.uint16), router, used)
    prob_all = prob_all.astype(np.float32)
    want = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x_all.view(np.uint16), prob_all, ids_all, threads=1)
    if bad:
        # a selection outside the expert table on every rank's share of the tokens: it adds nothing,
        # the token's sum is that of its other selections in their order
        ids_all = ids_all.copy()
        for t in range(1, tokens_all, 4):
            kept = np.ascontiguousarray(np.delete(ids_all[t], 1).reshape(1, used - 1))
            want[t] = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, x_all[t:t + 1].view(np.uint16),
                                     prob_all[t:t + 1], kept, threads=1)[0]
            ids_all[t, 1] = experts + 5
    t0, t1 = shard_rows(tokens_all, world, rank)
    e0, e1 = shard_rows(experts, world, rank)
    seen = []

    def run_experts(rows, local_expert):
        # rows that name one of this rank's experts are real; the others are padding of the
        # fixed-size exchange and their results are never read
        local = local_expert.numpy().astype(np.int64)
        real = (local >= 0) & (local < e1 - e0)
        seen.extend((local[real] + e0).tolist())
        out = np.zeros((rows.shape[0], hidden), np.float32)
        if real.any():
            ids = (local[real] + e0).astype(np.uint32).reshape(-1, 1)
            ones = np.ones((int(real.sum()), experts), np.float32)
            picked = np.ascontiguousarray(rows.numpy()[real])
            out[real] = oracle.moe_ffn(wg, wu, wd, experts, hidden, ffn, picked.view(np.uint16), ones, ids,
                                       threads=1)
        return torch.from_numpy(out)

    def combine(proj, prob, ids):
        # a selection that names no expert adds nothing: its projection rows are zero and its
        # weight is taken as that of expert 0, so the sum does not change... except that adding a
        # signed zero may not be the identity for -0.0; the kernel skips the rank instead
        picks = ids.numpy().view(np.uint32)
        out = np.zeros((proj.shape[0], proj.shape[2]), np.float32)
        for t in range(proj.shape[0]):
            good = [r for r in range(picks.shape[1]) if picks[t, r] < experts]
            one = np.ascontiguousarray(proj.numpy()[t:t + 1, good].transpose(1, 0, 2))
            out[t] = oracle.ordered_sum(one, prob.numpy()[t:t + 1], np.ascontiguousarray(picks[t:t + 1, good]))[0]
        return torch.from_numpy(out)

    ep = ExpertParallel(experts, used, hidden, world, rank, run_experts, combine)
    out = ep.ffn(torch.from_numpy(x_all[t0:t1]), torch.from_numpy(prob_all[t0:t1]),
                 torch.from_numpy(ids_all[t0:t1].view(np.int32)))
    ok = np.array_equal(out.numpy().view(np.uint32), want[t0:t1].view(np.uint32))
    ok = ok and all(e0 <= e < e1 for e in seen)
    result[rank] = bool(ok)
    dist.destroy_process_group()


def _spawn(worker, world, *args):
    import torch.multiprocessing as mp
    manager = mp.Manager()
    result = manager.dict()
    port = _free_port()
    mp.spawn(worker, args=(world, port) + args + (result,), nprocs=world, join=True)
    return dict(result)


def test_shard_rows_cover_and_owner_agrees():
    from aotx_b200.sharded import expert_owner, shard_rows
    for n in (1, 7, 128, 151936, 57344):
        for world in (1, 2, 3, 8):
            spans = [shard_rows(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    for experts, world in ((128, 8), (7, 3), (5, 2)):
        for e in range(experts):
            r = expert_owner(e, experts, world)
            first, last = shard_rows(experts, world, r)
            assert first <= e < last
    assert shard_rows(151936, 8, 3) == (3 * 18992, 4 * 18992)


@pytest.mark.parametrize("world,n", [(2, 96), (3, 100)])
def test_column_split_all_gather(world, n):
    result = _spawn(_column_worker, world, n, 64, 5)
    assert result == {r: True for r in range(world)}


@pytest.mark.parametrize("world,bad", [(2, False), (3, False), (2, True)])
def test_expert_parallel_all_to_all(world, bad):
    """`bad`: some selections name no expert; every rank drops them alike and the exchange keeps
    its fixed shape."""
    result = _spawn(_expert_worker, world, bad)
    assert result == {r: True for r in range(world)}
